"""ctypes signatures of the host library (csrc/host)."""
from ctypes import c_char_p, c_double, c_float, c_int, c_longlong, c_ulonglong, c_void_p, POINTER

SIGS = {}
