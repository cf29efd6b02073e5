from .continuous_count import continuous_count
from .swiglu import swiglu, swiglu_packed
