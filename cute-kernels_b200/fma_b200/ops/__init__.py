from .continuous_count import continuous_count
from .grouped_gemm import grouped_gemm
from .swiglu import swiglu, swiglu_packed
from .sequence_packing import pack_sequence, unpack_sequence
