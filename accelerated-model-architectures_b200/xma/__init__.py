"""B200-native implementation of the MoE hot path of XMA behind the reference's entry points:
`xma.layers.MoE`, `xma.functional.continuous_count`, `xma.functional.swiglu`, `xma.functional.swiglu_packed`.
Importing this package loads libxma_b200.so; it raises if the library has not been built."""

from . import _lib  # noqa: F401  (fails loudly when the CUDA library is missing)
from ._lib import check_device_status
from .accelerator import Accelerator, KernelBackend
from .utils import set_seed
from . import functional, layers  # noqa: E402
