"""get_mk / call_mk of the B200 route (the ctypes binding of libqmk_b200.so)."""
from qimeng_megakernel_b200.mk_kernel import MegaKernel, call_mk, get_mk  # noqa: F401
