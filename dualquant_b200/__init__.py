"""dualquant_b200: Blackwell-native (sm_100a) W4A4 inference hot path of DualQuant behind the
reference's PermLinear / FormatSpec Python API.  Compute lives in libdualquant_b200.so
(hand-written CUDA, C ABI in include/dualquant_b200.h); this package is the host-side mirror."""

__version__ = "0.1.0"
