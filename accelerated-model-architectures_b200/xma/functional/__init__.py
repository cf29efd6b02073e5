from .continuous_count import continuous_count
from .swiglu import swiglu, swiglu_chunked, swiglu_packed
from .fused_residual_add_rmsnorm import fused_residual_add_rmsnorm
