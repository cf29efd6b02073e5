from .continuous_count import continuous_count
from .swiglu import swiglu, swiglu_chunked, swiglu_packed
from .fused_residual_add_rmsnorm import fused_residual_add_rmsnorm
from .load_balancing_loss import load_balancing_loss
from .sequence_packing import pack_sequence, unpack_sequence
