"""ctypes binding of libfga.so, the C ABI declared in include/fga.h.

The library is built in-tree by build_native.py (nvcc, sm_100a only). There is no fallback: if the
shared object is missing or a call fails, an exception is raised.
"""
import ctypes
import os
from ctypes import c_char_p, c_int, c_int32, c_int64, c_size_t, c_uint64, c_void_p, POINTER

_HERE = os.path.dirname(os.path.realpath(__file__))
LIB_PATH = os.environ.get('FGA_LIB') or os.path.join(_HERE, 'libfga.so')  # FGA_LIB: another build of the same ABI

_lib = None


class FgaError(RuntimeError):
    """A libfga entry point returned a non-zero status."""


def lib():
    """The loaded library (loads on first use; raises if it was never built)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FgaError(f'{LIB_PATH} is missing: run `python build_native.py` (needs nvcc); '
                           'there is no CPU or PyTorch fallback for the fused kernels')
        _lib = ctypes.CDLL(LIB_PATH)
        _declare(_lib)
    return _lib


def _declare(l):
    vp, i, i64 = c_void_p, c_int, c_int64
    pp = POINTER(c_void_p)
    l.fga_version.restype = i
    l.fga_last_error.restype = c_char_p
    l.fga_sm_count.restype = i
    l.fga_launch_count.restype = c_uint64
    l.fga_symm_alloc.argtypes = [c_size_t, pp]
    l.fga_symm_export.argtypes = [vp, c_char_p]
    l.fga_symm_open.argtypes = [c_char_p, pp]
    l.fga_symm_close.argtypes = [vp]
    l.fga_symm_free.argtypes = [vp]
    l.fga_symm_vmm_size.argtypes = [c_size_t]
    l.fga_symm_vmm_size.restype = i64
    l.fga_symm_alloc_vmm.argtypes = [c_size_t, pp, POINTER(c_int)]
    l.fga_symm_open_vmm.argtypes = [i, c_size_t, pp]
    l.fga_symm_release_vmm.argtypes = [vp, c_size_t]
    l.fga_barrier.argtypes = [vp, vp, i, i, i, vp, i, vp, vp, c_uint64, vp]
    l.fga_gemm_push.argtypes = [vp, i, i, i, vp, i, vp, i, i, pp, i64, i, i, vp, c_uint64, vp]
    l.fga_gemm_recv.argtypes = [vp, i, i, vp, i, i, vp, vp, vp, vp, pp, i, i, i, i, i, i, vp, vp, vp,
                                c_uint64, vp]
    l.fga_gemm_push_gqa.argtypes = [vp, i, i, i, vp, vp, i, i, i, pp, i64, i, i, vp, c_uint64, vp]
    l.fga_gemm_recv_gqa.argtypes = [vp, i, vp, i, vp, vp, vp, vp, pp, i, i, i, i, i, i, i, i, vp, vp, c_uint64, vp]
    l.fga_gemm_local.argtypes = [vp, i, vp, i, i, i, i, i64, i64, vp, i64, i, i, vp, c_uint64, vp]
    l.fga_gemm_local_mx.argtypes = [vp, vp, i64, vp, vp, i64, i, i, i, vp, i64, i, i, vp, c_uint64, vp]
    l.fga_gemm_push_mx.argtypes = [vp, vp, i64, i, i, vp, vp, i64, vp, i, i, pp, i64, i, i, vp, c_uint64, vp]
    l.fga_gemm_recv_mx.argtypes = [vp, vp, vp, i, i, vp, vp, i64, i, i, vp, vp, vp, vp, pp, i, i, i, i, i, i,
                                   vp, vp, vp, c_uint64, vp]
    l.fga_gemm_push_gqa_mx.argtypes = [vp, vp, i64, i, i, vp, vp, i64, vp, i, i, i, pp, i64, i, i, vp, c_uint64, vp]
    l.fga_gemm_recv_gqa_mx.argtypes = [vp, vp, vp, i, vp, vp, i64, i, i, vp, vp, vp, vp, pp, i, i, i, i, i, i, i, i,
                                       vp, vp, c_uint64, vp]
    l.fga_copy_rank_rows.argtypes = [pp, pp, i, i, i64, i64, i, vp, i, i, vp]
    l.fga_bias_grad_scratch_floats.argtypes = [i64, i]
    l.fga_bias_grad_scratch_floats.restype = i64
    l.fga_bias_grad.argtypes = [vp, i64, i, vp, i, i, vp, vp]
    l.fga_bias_grad_static_capacity_floats.restype = i64
    l.fga_bias_grad_static.argtypes = [vp, i64, i, vp, i, i, vp]
    l.fga_mx_quantize.argtypes = [vp, i64, i, i64, i64, vp, vp, i64, i, vp]
    for name in ('fga_symm_alloc', 'fga_symm_export', 'fga_symm_open', 'fga_symm_close',
                 'fga_symm_free', 'fga_symm_alloc_vmm', 'fga_symm_open_vmm', 'fga_symm_release_vmm', 'fga_barrier', 'fga_gemm_push', 'fga_gemm_recv',
                 'fga_gemm_push_gqa', 'fga_gemm_recv_gqa',
                 'fga_gemm_local', 'fga_gemm_local_mx', 'fga_gemm_push_mx', 'fga_gemm_recv_mx',
                 'fga_gemm_push_gqa_mx', 'fga_gemm_recv_gqa_mx', 'fga_copy_rank_rows', 'fga_bias_grad', 'fga_bias_grad_static',
                 'fga_mx_quantize'):
        getattr(l, name).restype = i


EXPORTS = ('fga_version', 'fga_last_error', 'fga_sm_count', 'fga_launch_count', 'fga_symm_alloc', 'fga_symm_export',
           'fga_symm_open', 'fga_symm_close', 'fga_symm_free', 'fga_symm_vmm_size', 'fga_symm_alloc_vmm',
           'fga_symm_open_vmm', 'fga_symm_release_vmm', 'fga_barrier', 'fga_gemm_push',
           'fga_gemm_recv', 'fga_gemm_push_gqa', 'fga_gemm_recv_gqa', 'fga_gemm_local', 'fga_gemm_local_mx', 'fga_gemm_push_mx', 'fga_gemm_recv_mx',
           'fga_gemm_push_gqa_mx', 'fga_gemm_recv_gqa_mx', 'fga_copy_rank_rows', 'fga_bias_grad_scratch_floats',
           'fga_bias_grad', 'fga_bias_grad_static_capacity_floats', 'fga_bias_grad_static', 'fga_mx_quantize')


def check(rc, exc=FgaError):
    """Raise `exc` with the library's message when an entry point failed."""
    if rc != 0:
        message = lib().fga_last_error().decode(errors='replace')
        if rc == -1:
            raise ValueError(message)
        raise exc(f'libfga error {rc}: {message}')


def ptr_array(addresses):
    """A C array of void* from integer addresses."""
    arr = (c_void_p * len(addresses))(*addresses)
    return arr


DEVICE_ERRORS = {
    1: 'group barrier timed out: a CP peer never published its epoch',
    2: 'receive GEMM timed out: a row block never collected all peer arrivals',
    3: 'GEMM pipeline barrier timed out',
    4: 'receive-side quantizer timed out',
}
