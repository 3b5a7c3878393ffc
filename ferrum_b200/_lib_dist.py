"""ctypes signatures of the inter-GPU entry points (csrc/dist)."""
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p, POINTER

SIGS = {}
