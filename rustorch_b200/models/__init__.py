"""Model zoo (src/models/mod.rs): GPT-2 family, BERT, generic Transformer, ResNet / CNN, RNN / LSTM / Seq2Seq,
Keras-style Sequential and the save / load helpers."""
from .cnn import CNN, BasicBlock, Bottleneck, CNNBuilder, ResNet, ResNetBuilder, resnet18, resnet34, resnet50
from .gpt import GPT, GPTBlock, GPTConfig, gpt2_medium, gpt2_small
from .high_level import (BasicSequential, FitConfig, HighLevelModel, InferenceEngine, Metrics, Model, ModelBuilder, ModelConverter,
                         ModelInfo, ModelLoader, ModelMode, ModelSaver, Sequential, SerializationFormat, TrainingHistory,
                         count_parameters)
from .sequence import (BERT, BERTBuilder, BERTConfig, BERTEmbeddings, LSTMModel, LSTMModelBuilder, RNNModel, RNNModelBuilder,
                       Seq2SeqModel, Seq2SeqModelBuilder, TransformerModel, TransformerModelBuilder, bert_base_uncased,
                       bert_large_uncased)
