"""ctypes binding of libduq4.so (the C ABI declared in include/duq4.h).

The library is the product: there is no CPU or PyTorch fallback. Importing this module
when libduq4.so has not been built raises immediately (build it with
`python -m duqlinear4bitcuda_b200.build`).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libduq4.so")

MODE_NONE, MODE_SYM, MODE_SYM_DUAL, MODE_ASYM, MODE_ASYM_DUAL = 0, 1, 2, 3, 4
MODES = {"none": MODE_NONE, "sym": MODE_SYM, "sym_dual": MODE_SYM_DUAL, "asym": MODE_ASYM, "asym_dual": MODE_ASYM_DUAL}


class Epilogue(ctypes.Structure):
    """Mirror of `duq4_epilogue`."""
    _fields_ = [
        ("mode", ctypes.c_int32),
        ("col_offset", ctypes.c_uint32),
        ("scale_row", ctypes.c_void_p),
        ("zeros_row", ctypes.c_void_p),
        ("scale_col_1", ctypes.c_void_p),
        ("zeros_col_1", ctypes.c_void_p),
        ("scale_col_2", ctypes.c_void_p),
        ("zeros_col_2", ctypes.c_void_p),
        ("bias", ctypes.c_void_p),
        ("ldo", ctypes.c_uint32),
        ("n_out_peers", ctypes.c_uint32),
        ("out_peers", ctypes.c_void_p * 8),
        ("next_weights", ctypes.c_void_p),
        ("next_weights_bytes", ctypes.c_uint64),
        ("out_multicast", ctypes.c_void_p),
        ("n_acc_owners", ctypes.c_uint32),
        ("acc_rows_per_owner", ctypes.c_uint32),
        ("acc_slot", ctypes.c_uint32),
        ("acc_owners", ctypes.c_void_p * 8),
        ("out_rows_per_owner", ctypes.c_uint32),
    ]


class Duq4Error(RuntimeError):
    def __init__(self, fn, status, text):
        super().__init__(f"{fn} failed with status {status}: {text}")
        self.status = status


_vp, _u32, _f32, _sz, _i = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_float, ctypes.c_size_t, ctypes.c_int

# name -> argument types (return type is int unless listed in _RESTYPES)
SIGNATURES = {
    "duq4_version": [],
    "duq4_error_string": [_i],
    "duq4_dual_quant_col_k": [],
    "duq4_tensor_map_cache_entries": [],
    "duq4_set_static_weights": [_i],
    "duq4_sym_quant": [_vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_sym_dual_quant": [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_asym_quant": [_vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_asym_dual_quant": [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_asym_quant_8bit": [_vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "duq4_quantize_sym_fused": [_vp, _u32, _u32, _f32, _vp, _vp, _vp],
    "duq4_quantize_asym_fused": [_vp, _u32, _u32, _vp, _vp, _vp, _vp],
    "duq4_quantize_sym_dual_fused": [_vp, _u32, _u32, _f32, _vp, _vp, _vp, _vp],
    "duq4_quantize_asym_dual_fused": [_vp, _u32, _u32, _vp, _vp, _vp, _vp, _vp, _vp],
    "duq4_quantize_fused_i8": [_i, _vp, _u32, _u32, _f32, _vp, _vp, _vp, _vp, _vp, _vp],
    "duq4_silu_mul_quantize_fused": [_i, _vp, _u32, _u32, _u32, _u32, _f32, _vp, _i, _vp, _vp, _vp],
    "duq4_linear_w4a4_preunpacked": [_vp, _vp, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp, _vp],
    "duq4_weight_prelayout_i8": [_vp, _u32, _u32, _vp, _vp],
    "duq4_gemm_split_scratch_bytes": [],
    "duq4_linear_w4a4_prelaid": [_vp, _vp, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp, _vp, _sz, _vp],
    "duq4_linear_w4a4_from_fp16_prelaid": [_vp, _vp, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _vp, _vp, _sz, _vp],
    "duq4_sym_dequant": [_vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "duq4_sym_dual_dequant": [_vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "duq4_asym_dequant": [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "duq4_asym_dual_dequant": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "duq4_asym_batch_dequant": [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_asym_dequant_hprec": [_vp, _vp, _vp, _vp, _vp, _u32, _u32, _vp, _vp],
    "duq4_matmul_4bit": [_vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_matmul_8bit": [_vp, _vp, _u32, _u32, _u32, _vp, _vp],
    "duq4_batch_matmul_4bit": [_vp, _vp, _u32, _u32, _u32, _vp, _u32, _vp],
    "duq4_linear_w4a4": [_vp, _vp, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp, _vp],
    "duq4_linear_w4a4_batched": [_vp, _vp, _u32, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp, _vp],
    "duq4_linear_from_fp16_workspace_bytes": [_u32, _u32],
    "duq4_linear_from_fp16_prelaid_workspace_bytes": [_u32, _u32],
    "duq4_linear_w4a4_from_fp16": [_vp, _vp, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _vp, _vp, _sz, _vp],
    "duq4_linear_w4a4_gate_up_silu": [_vp, _i, _vp, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp],
    "duq4_linear_w4a4_gate_up_silu_prelaid": [_vp, _vp, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp],
    "duq4_linear_host_staging_bytes": [_u32, _u32, _u32, _u32],
    "duq4_linear_w4a4_from_fp16_host": [_vp, _vp, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _vp, _u32, _vp, _sz, _vp],
    "duq4_linear_pipeline_staging_bytes": [_i, _i, _u32, _u32, _u32, _u32],
    "duq4_linear_w4a4_from_fp16_to_host": [_vp, _vp, _i, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _vp, _u32, _vp, _sz, _vp],
    "duq4_linear_w4a4_from_fp16_to_peers": [_vp, _vp, _i, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _u32, _u32, _vp, _sz, _vp],
    "duq4_linear_w4a4_from_fp16_static": [_vp, _vp, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _vp, _vp],
    "duq4_row_stats": [_i, _vp, _u32, _u32, _vp, _vp, _vp],
    "duq4_quantize_i8_from_stats": [_i, _vp, _u32, _u32, _vp, _vp, _f32, _vp, _vp, _vp, _vp],
    "duq4_reduce_dequant_gather": [_vp, _u32, _u32, _u32, _u32, _u32, ctypes.POINTER(Epilogue), _vp, _vp],
    "duq4_linear_w4a4_from_fp16_to_host_rows": [_vp, _vp, _i, _u32, _u32, _u32, _i, _f32, ctypes.POINTER(Epilogue), _u32, _u32,
                                                ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_uint64), ctypes.c_uint64, _vp, _u32, _vp, _sz, _vp],
    "duq4_peer_barrier": [ctypes.POINTER(ctypes.c_void_p), _u32, _u32, ctypes.c_uint64, ctypes.c_uint64, _vp],
    "duq4_last_device_status": [_vp, ctypes.POINTER(ctypes.c_int32)],
}
_RESTYPES = {"duq4_version": ctypes.c_char_p, "duq4_error_string": ctypes.c_char_p,
             "duq4_linear_from_fp16_workspace_bytes": ctypes.c_size_t, "duq4_gemm_split_scratch_bytes": ctypes.c_size_t,
             "duq4_linear_from_fp16_prelaid_workspace_bytes": ctypes.c_size_t,
             "duq4_linear_host_staging_bytes": ctypes.c_size_t, "duq4_linear_pipeline_staging_bytes": ctypes.c_size_t}

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build the CUDA library first (python -m duqlinear4bitcuda_b200.build). "
        "There is no fallback path.")

cdll = ctypes.CDLL(LIB_PATH)
for _name, _args in SIGNATURES.items():
    _fn = getattr(cdll, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.argtypes = _args
    _fn.restype = _RESTYPES.get(_name, ctypes.c_int)


def check(fn_name, status):
    if status != 0:
        raise Duq4Error(fn_name, status, cdll.duq4_error_string(status).decode())


def call(fn_name, *args):
    """Call an int-returning entry point and raise Duq4Error on a non-zero status."""
    check(fn_name, getattr(cdll, fn_name)(*args))


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def current_stream():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def make_epilogue(mode, scale_row=None, zeros_row=None, scale_col_1=None, zeros_col_1=None, scale_col_2=None,
                  zeros_col_2=None, bias=None, col_offset=0, ldo=0, out_peers=None, next_weights=None, out_multicast=None,
                  acc_owners=None, acc_rows_per_owner=0, acc_slot=0, out_rows_per_owner=0):
    """Fill a duq4_epilogue. `next_weights`: packed weight tensor of the layer that runs next on the
    stream (L2 prefetch hint of the small-M kernels; never read or written by this launch)."""
    e = Epilogue()
    e.mode = MODES[mode] if isinstance(mode, str) else int(mode)
    e.col_offset = col_offset
    for k, v in (("scale_row", scale_row), ("zeros_row", zeros_row), ("scale_col_1", scale_col_1),
                 ("zeros_col_1", zeros_col_1), ("scale_col_2", scale_col_2), ("zeros_col_2", zeros_col_2),
                 ("bias", bias)):
        setattr(e, k, None if v is None else v.data_ptr())
    e.ldo = ldo
    if out_peers:   # raw device addresses (ints), this rank's own buffer included
        if len(out_peers) > 8:
            raise ValueError("at most 8 output peers")
        e.n_out_peers = len(out_peers)
        for i, a in enumerate(out_peers):
            e.out_peers[i] = int(a)
    if acc_owners:   # K-sharded layer: raw device addresses (ints) of every owner's int32 slab buffer
        e.n_acc_owners = len(acc_owners)
        e.acc_rows_per_owner = int(acc_rows_per_owner)
        e.acc_slot = int(acc_slot)
        for i, a in enumerate(acc_owners):
            e.acc_owners[i] = int(a)
    e.out_rows_per_owner = int(out_rows_per_owner)   # > 0: row m only to out_peers[m // out_rows_per_owner]
    if out_multicast:   # raw multicast address (int) of the same buffer, at this shard's first column
        e.out_multicast = int(out_multicast)
    if next_weights is not None:
        e.next_weights = next_weights.data_ptr()
        e.next_weights_bytes = next_weights.numel() * next_weights.element_size()
    return e
