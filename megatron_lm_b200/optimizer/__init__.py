from .optimizer import ChainedOptimizer, MixedPrecisionOptimizer, get_megatron_optimizer  # noqa: F401
from .grad_scaler import ConstantGradScaler, DynamicGradScaler  # noqa: F401
from .scheduler import OptimizerParamScheduler  # noqa: F401
