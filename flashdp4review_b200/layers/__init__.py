from .linear import DPLinear  # noqa: F401
from .layernorm import DPLayerNorm  # noqa: F401
from .transformers_conv1d import DPConv1D, Conv1D  # noqa: F401
from .utils import DPParameter  # noqa: F401
