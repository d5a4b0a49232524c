from .continuous_count import continuous_count
from .sequence_packing import pack_sequence, unpack_sequence
from .swiglu import swiglu
from .swiglu_packed import swiglu_packed
