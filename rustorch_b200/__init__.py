"""rustorch_b200: a Blackwell-native (sm_100a) deep-learning framework with the API surface of
RusTorch.  PyTorch is the tensor/autograd substrate; hot paths are hand-written CUDA kernels
(tcgen05 / TMEM / TMA) loaded from the in-tree ``_C`` extension.

The top-level names are those of the reference's Python bindings (python/src/lib.rs:44-1484 and
src/python/mod.rs:51-115): ``Tensor Variable Linear Conv2d ... SGD Adam tensor zeros ones no_grad grad``,
plus ``Device functional DataLoader Trainer DistributedDataParallel init_distributed ...``.  They resolve lazily,
so ``import rustorch_b200`` stays cheap.  ``import rustorch`` works through the alias package of the same tree.
"""
import importlib

from . import _native  # noqa: F401

__version__ = "0.1.0"


def native_available() -> bool:
    """True when the compiled sm_100a kernel library is importable."""
    return _native.available()


_LAZY = {
    # tensors / autograd
    "Tensor": "tensor", "tensor": "tensor", "zeros": "tensor", "ones": "tensor", "Variable": "autograd", "no_grad": "autograd",
    "enable_grad": "autograd", "grad": "autograd", "gradcheck": "autograd", "jacobian": "autograd", "hessian": "autograd",
    "Complex": "complex",
    **{n: "callbacks" for n in ("CallbackRegistry", "Result", "init_callback_system", "call_python_from_rust", "progress_callback_example",
                                "try_catch", "get_version", "hello_from_rust", "add_numbers", "sum_list")},
    # layers and losses
    **{n: "nn" for n in ("Module", "Parameter", "Sequential", "Linear", "Conv1d", "Conv2d", "Conv3d", "ConvTranspose2d", "MaxPool2d",
                         "AvgPool2d", "BatchNorm1d", "BatchNorm2d", "LayerNorm", "RMSNorm", "GroupNorm", "Dropout", "Flatten", "Embedding",
                         "ReLU", "Sigmoid", "Tanh", "GELU", "Softmax", "LeakyReLU", "MSELoss", "CrossEntropyLoss", "LSTM", "GRU", "RNN",
                         "MultiheadAttention", "Transformer", "TransformerEncoder", "TransformerEncoderLayer")},
    # optimizers / schedulers
    **{n: "optim" for n in ("SGD", "Adam", "AdamW", "RMSprop", "AdaGrad", "NAdam", "RAdam", "Adamax", "LAMB", "AdaBound", "LBFGS", "StepLR",
                            "ExponentialLR", "CosineAnnealingLR", "FusedAdamW", "FusedSGD")},
    # data / training / models
    **{n: "data" for n in ("Dataset", "TensorDataset", "DataLoader", "RandomSampler", "SequentialSampler", "BatchSampler")},
    **{n: "training" for n in ("Trainer", "TrainerConfig", "TrainerBuilder", "EarlyStopping", "CheckpointManager")},
    "TrainingHistory": "models.high_level", "Model": ("models.high_level", "BindingModel"), "ModelBuilder": "models.high_level",
    # utils of the binding
    **{n: "python_api" for n in ("Device", "Config", "ModelSerializer", "ModelComparator", "Transform", "Transforms", "DistributedConfig",
                                 "DistributedBackend",
                                 "init_distributed", "cleanup_distributed", "set_seed", "cuda_is_available", "get_system_info")},
    "Profiler": "profiler", "Plotter": "visualization", "ModelVisualizer": "visualization", "TensorStats": "visualization",
    # errors, hybrid f32 universe, parallel traits, hardware hints, misc named pieces
    **{n: "error" for n in ("RusTorchError", "RusTorchResult", "ShapeMismatch", "TensorOp", "GpuError", "DistributedError")},
    **{n: "hybrid_f32" for n in ("F32Tensor", "F32Variable", "F32Trainer", "F32TrainerConfig", "F32Linear", "F32Conv2d", "F32LSTM")},
    **{n: "parallel" for n in ("ParallelTensor", "ParallelConfig", "ParallelContext", "ParallelOp", "BatchParallelOp", "MatrixParallelOp",
                               "ReductionParallelOp", "SimdParallelOp", "batch_matmul_parallel", "kaiming_init")},
    **{n: "optimization" for n in ("HardwareOptimizer", "PlatformOptimizer", "SimdOptimizer")},
    **{n: "compat" for n in ("AdamConfig", "AdamState", "AdamUtils", "LBFGSMemory", "LineSearchMethod", "AllocationStrategy", "ZeroCopyOps",
                             "TensorIterOps", "ShapeBuilder", "LazyExpandedTensor", "SafeTensor", "SafeNumeric", "TypedTensor", "WindowType",
                             "Int4", "ProfilerCore", "RecurrentOps", "LinearBackward", "DistributedState", "GPTModel", "OnnxModel")},
    **{n: "compat_extra" for n in ("GradFn", "AddBackward", "SubBackward", "MulBackward", "MatMulBackward", "SumBackward", "MeanBackward",
                                   "TensorMetadata", "StateDict", "ModelStateDict", "AdamVariant", "CommonOps", "GenericAdamOptimizer",
                                   "GradientCompression", "GpuBuffer", "CudaBlas", "CudaSparseOps", "GpuActivation", "GpuConvolution",
                                   "GpuBatchMatrixExecutor", "CommunicationOp", "CommunicationManager", "get_compute_capability",
                                   "execute_attention")},
    **{n: "formats.loaders" for n in ("GGUFLoader", "SafetensorsLoader", "SafetensorsSaver", "Saver", "TensorLoader")},
    **{n: "gpu.devices" for n in ("GpuDevice", "GpuStream", "CpuDevice", "CudaDevice", "GpuKernel", "ModernGpuKernel", "AddKernel", "MatMulKernel",
                                  "ConvKernel", "KernelExecutor", "CudaKernelExecutor", "CudaMatrixExecutor", "CudaBuffer", "ComputeBackend",
                                  "CpuBackend", "GpuBackend", "BackendManager", "SelectionStrategy", "StreamOperation",
                                  "MetalKernelExecutor", "OpenClKernelExecutor", "OpenClMatrixExecutor", "CoreMLHybrid", "MacHybrid")},
    # distributed
    **{n: "distributed" for n in ("DistributedDataParallel", "DistributedSampler", "get_world_size", "get_rank",
                                  "is_master", "DataParallel")},
}
_SUBMODULES = ("nn", "optim", "data", "training", "models", "distributed", "formats", "llm", "amp", "profiler", "debug", "validation",
               "tensorboard", "visualization", "vision", "distributions", "special", "quantization", "sparse", "memory", "gpu", "execution",
               "model_import", "convert", "model_hub", "jit", "cli", "autograd", "ops", "utils", "parallel", "error", "hybrid_f32",
               "optimization", "compat", "compat_extra", "complex")


# functional activations and image transforms of the reference's Python module (src/python/nn.rs, src/python/data.rs)
_FUNCTIONAL = ("relu", "sigmoid", "tanh", "softmax", "gelu", "leaky_relu", "swish", "elu", "selu", "mish")
_TRANSFORMS = ("normalize", "resize", "random_crop", "random_horizontal_flip")


def __getattr__(name):
    if name in _FUNCTIONAL:
        from .nn import layers
        return getattr(layers, name)
    if name in _TRANSFORMS:
        from .python_api import Transforms
        return getattr(Transforms, name)
    if name == "functional":
        from .nn import functional
        return functional
    if name == "is_tensor":
        from .tensor import Tensor
        return lambda obj: isinstance(obj, Tensor)
    if name in _SUBMODULES:
        return importlib.import_module(f"{__name__}.{name}")
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(f"module '{__name__}' has no attribute '{name}'")
    mod, attr = mod if isinstance(mod, tuple) else (mod, name)      # (module, name there) when the two differ
    return getattr(importlib.import_module(f"{__name__}.{mod}"), attr)


def __dir__():
    return sorted(list(globals()) + list(_LAZY) + list(_SUBMODULES) + ["functional", "is_tensor"] + list(_FUNCTIONAL) + list(_TRANSFORMS))
