"""``rustorch.nn``: layers, activations, losses, transformer, recurrent nets (src/nn/mod.rs)."""
from . import fused  # noqa: F401
from .layers import *  # noqa: F401,F403
from .layers import Module, Parameter, Sequential
from .loss import *  # noqa: F401,F403
from .rnn import GRU, GRUCell, LSTM, LSTMCell, RNN, RNNCell
from .transformer import (CrossAttention, MultiheadAttention, SelfAttention, Transformer, TransformerDecoder,
                          TransformerDecoderLayer, TransformerEncoder, TransformerEncoderLayer)
from .pruning import Pruner, PruningAwareModule, PruningMask, PruningMethod, PruningSchedule, PruningStructure
from .quantization import (CalibrationMode, QuantizationAwareModule, QuantizationParams, QuantizationType, QuantizedTensor,
                           Quantizer)
from .safe_ops import SafeOps, TensorStats
from .conv_base import ConvOps, Validator, collect_conv_parameters
from .recurrent_common import (MultiLayerUtils, RecurrentConfig, RecurrentOps, TrainingMode,
                               collect_recurrent_parameters)
from . import functional  # noqa: E402,F401
