from .continuous_count import continuous_count
from .swiglu_packed import swiglu_packed
