"""``frankentorch_b200.optim``: optimizers, LR schedulers and the AMP gradient scaler (mirror of ft-optim)."""
from .optimizers import (ASGD, LBFGS, LBFGSLineSearch, SGD, Adadelta, Adagrad, Adam, Adamax, AdamW, Muon, NAdam, Optimizer, RAdam,
                         RMSprop, Rprop, SparseAdam)
from .schedulers import (ChainedScheduler, ConstantLR, CosineAnnealingLR, CosineAnnealingWarmRestarts, CyclicLR, CyclicLRMode,
                         ExponentialLR, GradScaler, LambdaLR, LinearLR, LRScheduler, MultiplicativeLR, MultiStepLR,
                         OneCycleLR, PolynomialLR, ReduceLROnPlateau, SchedulerState, SequentialLR, StepLR)
