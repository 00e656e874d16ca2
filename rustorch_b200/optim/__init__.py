"""``rustorch.optim``: optimizers, schedulers, utilities (src/optim/mod.rs)."""
from .flat import FlatParams, FusedAdamW, FusedSGD
from .lr_scheduler import (AnnealStrategy, CosineAnnealingLR, ExponentialLR, LRScheduler, MultiStepLR, OneCycleLR,
                           PlateauMode, PolynomialLR, ReduceLROnPlateau, StepLR, ThresholdMode, WarmupScheduler)
from .optimizers import (LAMB, LBFGS, SGD, AdaBound, AdaGrad, Adagrad, Adam, Adamax, AdamW, NAdam, RAdam, RMSprop)
from .utils import (OptimizerBenchmark, OptimizerFactory, OptimizerMetrics, StabilityConfig, clip_grad_norm,
                    clip_grad_value, grad_norm)
