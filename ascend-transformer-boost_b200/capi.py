"""ctypes bindings of libatb_b200.so (the declarations of include/atb_b200.h) and thin torch helpers.

The library is the product; this module is the Python-side mirror of the reference's test harness
entry (`OperationTorch.set_param / execute`, tests/apitest/opstest/python/operations/operation_test.py:66-110
of the reference).  There is no fallback: if the shared library is missing, importing fails.
"""
import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libatb_b200.so")

FP16, BF16, INT8 = 0, 1, 2
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_TMA_MMA, KERNEL_MLA_TC5 = 0, 1, 2, 3
DTYPE_CODE = {"fp16": FP16, "bf16": BF16, "int8": INT8}

# aclDataType / aclFormat values (include/acl/acl.h)
ACL_FLOAT, ACL_FLOAT16, ACL_INT8, ACL_INT32, ACL_INT64, ACL_BF16 = 0, 1, 2, 3, 9, 27
ACL_FORMAT_ND = 2

# atb::ErrorType (include/atb/types.h)
NO_ERROR = 0
ERROR_INVALID_PARAM = 1
ERROR_RT_FAIL = 4
ERROR_INVALID_IN_TENSOR_NUM = 5
ERROR_INVALID_TENSOR_DIM = 8
ERROR_INVALID_TENSOR_SIZE = 9
ERROR_INVALID_TENSOR_INI_MATCH = 13
ERROR_INVALID_TENSOR_ADDR = 14
ERROR_INVALID_TENSOR_DIM_NUM = 16


class PaDesc(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int32), ("num_heads", ctypes.c_int32), ("kv_heads", ctypes.c_int32),
                ("head_dim_k", ctypes.c_int32), ("head_dim_v", ctypes.c_int32), ("v_row_dim", ctypes.c_int32),
                ("block_size", ctypes.c_int32), ("num_blocks", ctypes.c_int32),
                ("max_blocks_per_seq", ctypes.c_int32), ("q_dtype", ctypes.c_int32), ("kv_dtype", ctypes.c_int32),
                ("qk_scale", ctypes.c_float), ("kernel", ctypes.c_int32), ("sm_count", ctypes.c_int32),
                ("rope_dim", ctypes.c_int32), ("score_mods", ctypes.c_int32), ("kv_layout", ctypes.c_int32), ("q_per_seq", ctypes.c_int32),
                ("qkv_quant", ctypes.c_int32), ("out_dtype", ctypes.c_int32)]


class PaTensors(ctypes.Structure):
    _fields_ = [("q", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("block_tables", ctypes.c_void_p), ("k_descale", ctypes.c_void_p), ("v_descale", ctypes.c_void_p),
                ("k_offset", ctypes.c_void_p), ("v_offset", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("q_rope", ctypes.c_void_p), ("k_rope_cache", ctypes.c_void_p),
                ("mask", ctypes.c_void_p), ("mask_batch_stride", ctypes.c_int64), ("mask_head_stride", ctypes.c_int64),
                ("mask_tokens", ctypes.c_int64), ("mask_q_stride", ctypes.c_int64), ("logn", ctypes.c_void_p),
                ("lse_out", ctypes.c_void_p), ("p_scale", ctypes.c_void_p)]


QUANT_ONLINE, QUANT_OFFLINE = 1, 2
SCORE_MASK, SCORE_LOGN, SCORE_ROWS, SCORE_CAUSAL = 1, 2, 4, 8


class PaPlanInfo(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_int32), ("num_ctas", ctypes.c_int32), ("num_items", ctypes.c_int32),
                ("num_partials", ctypes.c_int32), ("num_combine_seqs", ctypes.c_int32),
                ("tile_tokens", ctypes.c_int32), ("workspace_bytes", ctypes.c_uint64),
                ("plan_bytes", ctypes.c_uint64), ("kernels_per_launch", ctypes.c_int32),
                ("reserved", ctypes.c_int32)]


class PaPeers(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("total_heads", ctypes.c_int32),
                ("head_offset", ctypes.c_int32), ("peer_out", ctypes.c_void_p * 8),
                ("peer_flags", ctypes.c_void_p * 8), ("epoch", ctypes.c_uint32), ("poll_limit", ctypes.c_uint32)]


class AtbTensor(ctypes.Structure):
    _fields_ = [("dtype", ctypes.c_int32), ("format", ctypes.c_int32), ("dims", ctypes.c_int64 * 8),
                ("dim_num", ctypes.c_uint64), ("device_data", ctypes.c_void_p), ("host_data", ctypes.c_void_p),
                ("data_size", ctypes.c_uint64)]


class PagedAttentionParam(ctypes.Structure):
    """Byte layout of atb::infer::PagedAttentionParam (120 bytes)."""
    _fields_ = [("headNum", ctypes.c_int32), ("qkScale", ctypes.c_float), ("kvHeadNum", ctypes.c_int32),
                ("maskType", ctypes.c_int32), ("batchRunStatusEnable", ctypes.c_bool), ("quantType", ctypes.c_int32),
                ("outDataType", ctypes.c_int32), ("hasQuantOffset", ctypes.c_bool), ("compressType", ctypes.c_int32),
                ("calcType", ctypes.c_int32), ("scaleType", ctypes.c_int32), ("inputLayout", ctypes.c_int32),
                ("mlaVHeadSize", ctypes.c_uint32), ("qScale", ctypes.c_float), ("rsv", ctypes.c_uint8 * 64)]

    def __init__(self, **kw):
        super().__init__()
        self.qkScale = 1.0
        self.outDataType = -1
        for k, v in kw.items():
            setattr(self, k, v)


class ReshapeAndCacheParam(ctypes.Structure):
    """Byte layout of atb::infer::ReshapeAndCacheParam (24 bytes)."""
    _fields_ = [("compressType", ctypes.c_int32), ("kvCacheCfg", ctypes.c_int32), ("rsv", ctypes.c_uint8 * 16)]


class ReshapeAndCacheWithStrideParam(ctypes.Structure):
    """Byte layout of atb::infer::ReshapeAndCacheWithStrideParam (24 bytes)."""
    _fields_ = [("compressType", ctypes.c_int32), ("kvCacheCfg", ctypes.c_int32), ("rsv", ctypes.c_uint8 * 16)]


class KvCacheParam(ctypes.Structure):
    """Byte layout of atb::infer::KvCacheParam (8 bytes)."""
    _fields_ = [("rsv", ctypes.c_uint8 * 8)]


class MultiLatentAttentionParam(ctypes.Structure):
    """Byte layout of atb::infer::MultiLatentAttentionParam (64 bytes); cacheMode 1 = separate latent / rope caches."""
    _fields_ = [("headNum", ctypes.c_int32), ("qkScale", ctypes.c_float), ("kvHeadNum", ctypes.c_int32),
                ("maskType", ctypes.c_int32), ("calcType", ctypes.c_int32), ("cacheMode", ctypes.c_uint8),
                ("windowSize", ctypes.c_uint32), ("maskUseStatusType", ctypes.c_int32), ("rsv", ctypes.c_uint8 * 32)]

    def __init__(self, **kw):
        super().__init__()
        self.qkScale = 1.0
        for k, v in kw.items():
            setattr(self, k, v)


class NormRopeReshapeParam(ctypes.Structure):
    """Byte layout of atb::infer::NormRopeReshapeParam (28 bytes)."""
    _fields_ = [("precisionMode", ctypes.c_uint32), ("rotaryCoeff", ctypes.c_uint32), ("epsilon", ctypes.c_float),
                ("rsv", ctypes.c_uint8 * 16)]

    def __init__(self, **kw):
        super().__init__()
        self.rotaryCoeff = 2
        self.epsilon = 1e-5
        for k, v in kw.items():
            setattr(self, k, v)


class BlockCopyParam(ctypes.Structure):
    """Byte layout of atb::infer::BlockCopyParam (16 bytes)."""
    _fields_ = [("rsv", ctypes.c_uint8 * 16)]


class PagedCacheLoadParam(ctypes.Structure):
    """Byte layout of atb::infer::PagedCacheLoadParam (64 bytes); kvCacheCfg 1 = ND caches."""
    _fields_ = [("kvCacheCfg", ctypes.c_int8), ("isSeqLensCumsumMode", ctypes.c_bool), ("hasSeqStarts", ctypes.c_bool),
                ("rsv", ctypes.c_uint8 * 61)]


# every symbol include/atb_b200.h declares
EXPORTS = [
    "atb_b200_pa_plan_create", "atb_b200_pa_plan_update", "atb_b200_pa_plan_set_rows", "atb_b200_pa_plan_get_info", "atb_b200_pa_plan_dump",
    "atb_b200_pa_plan_destroy", "atb_b200_pa_launch", "atb_b200_reshape_and_cache",
    "atb_b200_pa_plan_device_status", "atb_b200_pa_plan_set_profiling", "atb_b200_pa_plan_kernel_ms",
    "atb_b200_context_create", "atb_b200_context_set_stream", "atb_b200_context_destroy",
    "atb_b200_operation_create_paged_attention", "atb_b200_operation_create_reshape_and_cache",
    "atb_b200_operation_input_num", "atb_b200_operation_output_num", "atb_b200_operation_infer_shape",
    "atb_b200_operation_setup", "atb_b200_operation_execute", "atb_b200_operation_destroy", "atb_b200_version",
    "atb_b200_pa_decode_static_scratch", "atb_b200_pa_static_scratch_status", "atb_b200_pa_launch_gathered", "atb_b200_peer_buffer_create",
    "atb_b200_peer_buffer_open", "atb_b200_peer_buffer_close", "atb_b200_peer_buffer_destroy",
    "atb_b200_pa_plan_set_trace", "atb_b200_pa_plan_prefetch", "atb_b200_operation_name",
    "atb_b200_block_copy", "atb_b200_paged_cache_load", "atb_b200_paged_cache_load_workspace_bytes",
    "atb_b200_operation_create_block_copy", "atb_b200_operation_create_paged_cache_load",
    "atb_b200_reshape_and_cache_strided", "atb_b200_operation_create_reshape_and_cache_with_stride",
    "atb_b200_norm_rope_reshape", "atb_b200_operation_create_norm_rope_reshape",
    "atb_b200_operation_create_multi_latent_attention",
    "atb_b200_kv_cache", "atb_b200_operation_create_kv_cache", "atb_b200_context_set_gather",
]

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python {_PKG}/build.py` "
                              "(there is no CPU or PyTorch fallback)")
        L = ctypes.CDLL(LIB_PATH)
        vp, i32, i64, u32, u64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_uint32, ctypes.c_uint64
        P = ctypes.POINTER
        L.atb_b200_pa_plan_create.argtypes = [P(PaDesc), vp, P(vp)]
        L.atb_b200_pa_plan_update.argtypes = [vp, vp]
        L.atb_b200_pa_plan_set_rows.argtypes = [vp, vp, ctypes.c_int32, vp, ctypes.c_int64]
        L.atb_b200_pa_plan_get_info.argtypes = [vp, P(PaPlanInfo)]
        L.atb_b200_pa_plan_dump.argtypes = [vp, vp, i32, vp, i32]
        L.atb_b200_pa_plan_destroy.argtypes = [vp]
        L.atb_b200_pa_plan_destroy.restype = None
        L.atb_b200_pa_launch.argtypes = [vp, P(PaTensors), vp, u64, vp]
        L.atb_b200_reshape_and_cache.argtypes = [vp, vp, vp, vp, vp, i32, i64, i64, i64, vp]
        L.atb_b200_pa_plan_device_status.argtypes = [vp, vp, vp, P(i32)]
        L.atb_b200_pa_plan_set_profiling.argtypes = [vp, ctypes.c_int]
        L.atb_b200_pa_plan_kernel_ms.argtypes = [vp, i32, P(ctypes.c_float)]
        L.atb_b200_context_create.argtypes = [P(vp)]
        L.atb_b200_context_set_stream.argtypes = [vp, vp]
        L.atb_b200_context_destroy.argtypes = [vp]
        L.atb_b200_operation_create_paged_attention.argtypes = [vp, u64, P(vp)]
        L.atb_b200_operation_create_reshape_and_cache.argtypes = [vp, u64, P(vp)]
        L.atb_b200_operation_create_block_copy.argtypes = [vp, u64, P(vp)]
        L.atb_b200_operation_create_multi_latent_attention.argtypes = [vp, u64, P(vp)]
        L.atb_b200_operation_create_kv_cache.argtypes = [vp, u64, P(vp)]
        L.atb_b200_kv_cache.argtypes = [vp, vp, vp, vp, vp, ctypes.c_int64, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                        ctypes.c_int64, vp]
        L.atb_b200_operation_create_norm_rope_reshape.argtypes = [vp, u64, P(vp)]
        L.atb_b200_norm_rope_reshape.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, ctypes.c_float, i64, vp]
        L.atb_b200_operation_create_reshape_and_cache_with_stride.argtypes = [vp, u64, P(vp)]
        L.atb_b200_reshape_and_cache_strided.argtypes = [vp, vp, vp, vp, vp, i32, i64, i64, i64, i64, i64, vp]
        L.atb_b200_operation_create_paged_cache_load.argtypes = [vp, u64, P(vp)]
        L.atb_b200_operation_input_num.argtypes = [vp, P(u32)]
        L.atb_b200_operation_output_num.argtypes = [vp, P(u32)]
        L.atb_b200_operation_infer_shape.argtypes = [vp, P(AtbTensor), u32, P(AtbTensor), u32]
        L.atb_b200_operation_setup.argtypes = [vp, P(AtbTensor), u32, P(AtbTensor), u32, P(u64), vp]
        L.atb_b200_operation_execute.argtypes = [vp, P(AtbTensor), u32, P(AtbTensor), u32, vp, u64, vp]
        L.atb_b200_operation_destroy.argtypes = [vp]
        L.atb_b200_operation_name.argtypes = [vp, ctypes.c_char_p, u64]
        L.atb_b200_version.restype = ctypes.c_char_p
        L.atb_b200_pa_decode_static_scratch.argtypes = [P(PaDesc), vp, P(PaTensors), vp]
        L.atb_b200_pa_static_scratch_status.argtypes = [vp, P(ctypes.c_int32)]
        L.atb_b200_pa_launch_gathered.argtypes = [vp, P(PaTensors), P(PaPeers), vp, u64, vp]
        L.atb_b200_context_set_gather.argtypes = [vp, P(PaPeers)]
        L.atb_b200_peer_buffer_create.argtypes = [u64, P(vp), ctypes.c_char_p]
        L.atb_b200_peer_buffer_open.argtypes = [ctypes.c_char_p, P(vp)]
        L.atb_b200_peer_buffer_close.argtypes = [vp]
        L.atb_b200_peer_buffer_destroy.argtypes = [vp]
        L.atb_b200_pa_plan_set_trace.argtypes = [vp, vp, u32]
        L.atb_b200_pa_plan_prefetch.argtypes = [vp, vp]
        L.atb_b200_block_copy.argtypes = [vp, vp, vp, vp, vp, i32, i32, i64, i64, i64, vp]
        L.atb_b200_paged_cache_load_workspace_bytes.argtypes = [i32, i32]
        L.atb_b200_paged_cache_load_workspace_bytes.restype = u64
        L.atb_b200_paged_cache_load.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i64, i64, i64, i64, i32, vp,
                                                u64, vp]
        _lib = L
    return _lib


class AtbError(RuntimeError):
    def __init__(self, what, code):
        super().__init__(f"{what} failed with atb::ErrorType {code}")
        self.code = code


def _check(rc, what):
    if rc != 0:
        raise AtbError(what, rc)


# ------------------------------------------------------------------ kernel level

def make_desc(batch, num_heads, kv_heads, dk, dv, block_size, num_blocks, max_blocks, q_dtype, kv_dtype=None,
              qk_scale=1.0, v_row_dim=None, kernel=KERNEL_AUTO, sm_count=0, rope_dim=0, score_mods=0, kv_layout=0, q_per_seq=0,
              qkv_quant=0, out_dtype=None):
    d = PaDesc()
    d.q_per_seq = q_per_seq
    d.qkv_quant = qkv_quant
    d.out_dtype = 0 if out_dtype is None else (DTYPE_CODE[out_dtype] if isinstance(out_dtype, str) else out_dtype)
    d.rope_dim, d.score_mods, d.kv_layout = rope_dim, score_mods, kv_layout
    d.batch, d.num_heads, d.kv_heads = batch, num_heads, kv_heads
    d.head_dim_k, d.head_dim_v, d.v_row_dim = dk, dv, (v_row_dim or dv)
    d.block_size, d.num_blocks, d.max_blocks_per_seq = block_size, num_blocks, max_blocks
    d.q_dtype = DTYPE_CODE[q_dtype] if isinstance(q_dtype, str) else q_dtype
    kv = kv_dtype or q_dtype
    d.kv_dtype = DTYPE_CODE[kv] if isinstance(kv, str) else kv
    d.qk_scale, d.kernel, d.sm_count = qk_scale, kernel, sm_count
    return d


class PaPlan:
    """Owns an atb_b200_pa_plan.  `context_lens` is a host int32 numpy array."""

    def __init__(self, desc, context_lens):
        import numpy as np
        self._lens = np.ascontiguousarray(context_lens, dtype=np.int32)
        self.desc = desc
        self.handle = ctypes.c_void_p()
        _check(lib().atb_b200_pa_plan_create(ctypes.byref(desc), self._lens.ctypes.data, ctypes.byref(self.handle)),
               "atb_b200_pa_plan_create")

    def update(self, context_lens):
        import numpy as np
        self._lens = np.ascontiguousarray(context_lens, dtype=np.int32)
        _check(lib().atb_b200_pa_plan_update(self.handle, self._lens.ctypes.data), "atb_b200_pa_plan_update")

    def set_rows(self, bt_rows, bt_row_count, mask_rows=None, mask_row_count=0):
        """SCORE_ROWS plans: the block-table row and the mask row of every query token (host int32 arrays)."""
        import numpy as np
        bt = np.ascontiguousarray(bt_rows, dtype=np.int32)
        mr = None if mask_rows is None else np.ascontiguousarray(mask_rows, dtype=np.int32)
        _check(lib().atb_b200_pa_plan_set_rows(self.handle, bt.ctypes.data, int(bt_row_count),
                                               None if mr is None else mr.ctypes.data, int(mask_row_count)),
               "atb_b200_pa_plan_set_rows")

    @property
    def info(self):
        info = PaPlanInfo()
        _check(lib().atb_b200_pa_plan_get_info(self.handle, ctypes.byref(info)), "atb_b200_pa_plan_get_info")
        return info

    def dump(self):
        import numpy as np
        info = self.info
        items = np.zeros((max(info.num_items, 1), 4), dtype=np.int32)
        groups = np.zeros(info.num_ctas + 2, dtype=np.int32)
        _check(lib().atb_b200_pa_plan_dump(self.handle, items.ctypes.data, items.shape[0], groups.ctypes.data,
                                           groups.shape[0]), "atb_b200_pa_plan_dump")
        return items[:info.num_items], groups

    def launch(self, tensors, workspace_ptr, workspace_bytes, stream_ptr):
        _check(lib().atb_b200_pa_launch(self.handle, ctypes.byref(tensors), workspace_ptr, workspace_bytes,
                                        stream_ptr), "atb_b200_pa_launch")

    def launch_gathered(self, tensors, peers, workspace_ptr, workspace_bytes, stream_ptr):
        _check(lib().atb_b200_pa_launch_gathered(self.handle, ctypes.byref(tensors), ctypes.byref(peers),
                                                 workspace_ptr, workspace_bytes, stream_ptr),
               "atb_b200_pa_launch_gathered")

    def device_status(self, workspace_ptr, stream_ptr):
        st = ctypes.c_int32(-1)
        _check(lib().atb_b200_pa_plan_device_status(self.handle, workspace_ptr, stream_ptr, ctypes.byref(st)),
               "atb_b200_pa_plan_device_status")
        return st.value

    def prefetch(self, stream_ptr):
        _check(lib().atb_b200_pa_plan_prefetch(self.handle, stream_ptr), "atb_b200_pa_plan_prefetch")

    def set_trace(self, device_ptr, capacity):
        _check(lib().atb_b200_pa_plan_set_trace(self.handle, device_ptr, capacity), "atb_b200_pa_plan_set_trace")

    def set_profiling(self, on=True):
        """on: False / True (every launch) or a stride n (every n-th launch carries the event pair)."""
        _check(lib().atb_b200_pa_plan_set_profiling(self.handle, int(on)), "atb_b200_pa_plan_set_profiling")

    def kernel_ms(self, launches_back=0):
        """Duration of the attention kernel `launches_back` launches ago (profiling must be on)."""
        ms = ctypes.c_float(0)
        _check(lib().atb_b200_pa_plan_kernel_ms(self.handle, launches_back, ctypes.byref(ms)),
               "atb_b200_pa_plan_kernel_ms")
        return ms.value

    def close(self):
        if self.handle:
            lib().atb_b200_pa_plan_destroy(self.handle)
            self.handle = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def torch_stream_ptr():
    import torch
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def pa_tensors(q, k_cache, v_cache, block_tables, out, k_descale=None, v_descale=None, k_offset=None, v_offset=None,
               q_rope=None, k_rope_cache=None, mask=None, mask_strides=(0, 0), mask_tokens=0, logn=None, lse_out=None, mask_q_stride=0,
               p_scale=None):
    """`mask_strides` = (batch, head) element strides of the additive mask, `mask_tokens` its last dimension."""
    t = PaTensors()
    t.p_scale = _ptr(p_scale)
    t.mask, t.logn, t.lse_out = _ptr(mask), _ptr(logn), _ptr(lse_out)
    t.mask_q_stride = int(mask_q_stride)
    t.mask_batch_stride, t.mask_head_stride, t.mask_tokens = int(mask_strides[0]), int(mask_strides[1]), int(mask_tokens)
    t.q_rope, t.k_rope_cache = _ptr(q_rope), _ptr(k_rope_cache)
    t.q, t.k_cache = _ptr(q), _ptr(k_cache)
    t.v_cache = _ptr(v_cache if v_cache is not None else k_cache)
    t.block_tables, t.out = _ptr(block_tables), _ptr(out)
    t.k_descale, t.v_descale, t.k_offset, t.v_offset = _ptr(k_descale), _ptr(v_descale), _ptr(k_offset), _ptr(v_offset)
    return t


def paged_attention(q, k_cache, v_cache, block_tables, context_lens_host, qk_scale, dv=None, k_descale=None,
                    v_descale=None, k_offset=None, v_offset=None, out=None, kernel=KERNEL_AUTO, plan=None,
                    workspace=None, return_plan=False):
    """One decode step on torch CUDA tensors through the kernel-level C ABI (plan + launch).

    v_cache=None selects the combined (MLA) cache: V = K[..., :dv].
    """
    import torch
    name = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.int8: "int8"}
    B, H, Dk = q.shape
    NB, BS, Hkv, _ = k_cache.shape
    if v_cache is None:
        v_row, dv = Dk, dv
    else:
        v_row = v_cache.shape[3]
        dv = dv or v_row
    if out is None:
        out = torch.zeros((B, H, dv), dtype=q.dtype, device=q.device)
    if plan is None:
        desc = make_desc(B, H, Hkv, Dk, dv, BS, NB, block_tables.shape[1], name[q.dtype], name[k_cache.dtype],
                         qk_scale, v_row_dim=v_row, kernel=kernel)
        plan = PaPlan(desc, context_lens_host)
    info = plan.info
    if workspace is None or workspace.numel() < info.workspace_bytes:
        workspace = torch.empty(max(int(info.workspace_bytes), 256), dtype=torch.uint8, device=q.device)
    t = pa_tensors(q, k_cache, v_cache, block_tables, out, k_descale, v_descale, k_offset, v_offset)
    plan.launch(t, ctypes.c_void_p(workspace.data_ptr()), workspace.numel(), torch_stream_ptr())
    if return_plan:
        return out, plan, workspace
    return out


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping):
    """In-place scatter of the new tokens into the caches (value / value_cache may be None)."""
    n = key.shape[0]
    krow = key[0].numel() * key.element_size() if n else 0
    vrow = value[0].numel() * value.element_size() if (value is not None and n) else 0
    nslots = key_cache.shape[0] * key_cache.shape[1]
    _check(lib().atb_b200_reshape_and_cache(_ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache),
                                            _ptr(slot_mapping), n, krow, vrow, nslots, torch_stream_ptr()),
           "atb_b200_reshape_and_cache")


def block_copy(k_cache, v_cache, src_blocks, dst_blocks, cum_sum, stream_ptr=None):
    """In place on torch CUDA tensors: caches [blocks, block_size, heads, D]; int32 index tensors on the device."""
    kb = k_cache[0].numel() * k_cache.element_size()
    vb = v_cache[0].numel() * v_cache.element_size() if v_cache is not None else 0
    _check(lib().atb_b200_block_copy(_ptr(k_cache), _ptr(v_cache), _ptr(src_blocks), _ptr(dst_blocks), _ptr(cum_sum),
                                     src_blocks.numel(), dst_blocks.numel(), kb, vb, k_cache.shape[0],
                                     stream_ptr if stream_ptr is not None else torch_stream_ptr()), "atb_b200_block_copy")


def kv_cache(new_kv, layer_id, past, token_offset, seq_len, stream_ptr=None):
    """In place on torch CUDA tensors: past [layers, batch, max_seqlen, hidden] receives the rows of new_kv
    [tokens, hidden]; layer_id [1], token_offset [batch], seq_len [batch] are int32 device tensors."""
    _check(lib().atb_b200_kv_cache(_ptr(new_kv), _ptr(layer_id), _ptr(past), _ptr(token_offset), _ptr(seq_len),
                                   new_kv.shape[0], past.shape[0], past.shape[1], past.shape[2],
                                   past.shape[3] * past.element_size(),
                                   stream_ptr if stream_ptr is not None else torch_stream_ptr()), "atb_b200_kv_cache")


def paged_cache_load(k_cache, v_cache, block_tables, context_lens, key, value, seq_starts=None, cumulative=False,
                     stream_ptr=None):
    """Gathers cached tokens into key / value ([rows, heads, D] torch CUDA tensors)."""
    import torch
    batch = context_lens.numel() - (1 if cumulative else 0)
    ws_bytes = lib().atb_b200_paged_cache_load_workspace_bytes(batch, int(cumulative))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=key.device)
    _check(lib().atb_b200_paged_cache_load(
        _ptr(k_cache), _ptr(v_cache), _ptr(block_tables), _ptr(context_lens), _ptr(seq_starts), _ptr(key), _ptr(value),
        batch, block_tables.shape[1], k_cache.shape[1], k_cache[0, 0].numel() * k_cache.element_size(),
        v_cache[0, 0].numel() * v_cache.element_size() if v_cache is not None else 0, k_cache.shape[0], key.shape[0],
        int(cumulative), ws.data_ptr(), ws_bytes, stream_ptr if stream_ptr is not None else torch_stream_ptr()),
        "atb_b200_paged_cache_load")
    return ws


class PeerExchange:
    """Gathered-output buffers and flag arrays shared by the ranks of a node over CUDA IPC.

    Every rank creates `n_buffers` gathered output buffers of `out_bytes` and one flag array, hands
    the IPC handles to its peers through torch.distributed (any host channel would do) and maps
    theirs.  `peers(i)` builds the atb_b200_pa_peers argument of the i-th call.
    """

    def __init__(self, out_bytes, total_heads, head_offset, n_buffers=2):
        import torch.distributed as dist
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.total_heads, self.head_offset = total_heads, head_offset
        self.local, handles = [], []
        for _ in range(n_buffers + 1):                       # last one = the flag array
            ptr = ctypes.c_void_p()
            h = ctypes.create_string_buffer(64)
            nbytes = out_bytes if len(self.local) < n_buffers else 256
            _check(lib().atb_b200_peer_buffer_create(nbytes, ctypes.byref(ptr), h), "atb_b200_peer_buffer_create")
            self.local.append(ptr.value)
            handles.append(bytes(h.raw))
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handles)
        self.mapped = []                                      # [buffer][rank] -> pointer valid in this process
        self._opened = []
        for b in range(n_buffers + 1):
            row = []
            for r in range(self.world):
                if r == self.rank:
                    row.append(self.local[b])
                else:
                    p = ctypes.c_void_p()
                    _check(lib().atb_b200_peer_buffer_open(everyone[r][b], ctypes.byref(p)),
                           "atb_b200_peer_buffer_open")
                    row.append(p.value)
                    self._opened.append(p.value)
            self.mapped.append(row)
        self.n_buffers = n_buffers
        self.calls = 0
        self._structs = []
        for b in range(n_buffers):
            p = PaPeers()
            p.world, p.rank, p.total_heads, p.head_offset = self.world, self.rank, self.total_heads, self.head_offset
            for r in range(self.world):
                p.peer_out[r] = self.mapped[b][r]
                p.peer_flags[r] = self.mapped[n_buffers][r]
            self._structs.append(p)
        dist.barrier()

    def peers(self):
        """Argument for the next call: alternates the gathered buffer, advances the epoch.
        Returns (atb_b200_pa_peers, local pointer of the gathered buffer this call fills)."""
        b = self.calls % self.n_buffers
        self.calls += 1
        p = self._structs[b]
        p.epoch = self.calls
        return p, self.local[b]

    def local_tensor(self, ptr, shape, dtype):
        """A torch view of one of this rank's gathered buffers."""
        import torch
        nbytes = 1
        for s_ in shape:
            nbytes *= s_
        nbytes *= torch.empty((), dtype=dtype).element_size()

        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        return torch.as_tensor(raw, device="cuda").view(dtype).view(shape)

    def close(self):
        import torch.distributed as dist
        dist.barrier()
        for p in self._opened:
            lib().atb_b200_peer_buffer_close(p)
        self._opened = []
        dist.barrier()
        for p in self.local:
            lib().atb_b200_peer_buffer_destroy(p)
        self.local = []


# ------------------------------------------------------------------ operator level

def atb_tensor(t=None, *, dtype=None, shape=None, host=None, device_ptr=None, fmt=ACL_FORMAT_ND):
    """Builds an atb::Tensor view of a torch tensor (or of an explicit dtype/shape for negative tests)."""
    a = AtbTensor()
    if t is not None:
        import torch
        code = {torch.float16: ACL_FLOAT16, torch.bfloat16: ACL_BF16, torch.int8: ACL_INT8, torch.int32: ACL_INT32,
                torch.float32: ACL_FLOAT, torch.int64: ACL_INT64}[t.dtype]
        shape = tuple(t.shape)
        a.dtype = code if dtype is None else dtype
        a.device_data = t.data_ptr() if t.is_cuda else None
        a.data_size = t.numel() * t.element_size()
        if not t.is_cuda:
            a.host_data = t.data_ptr()
    else:
        a.dtype = dtype
        size = {ACL_FLOAT16: 2, ACL_BF16: 2, ACL_INT8: 1, ACL_INT32: 4, ACL_FLOAT: 4, ACL_INT64: 8}.get(dtype, 1)
        n = 1
        for s in shape:
            n *= s
        a.data_size = n * size
        a.device_data = device_ptr
    a.format = fmt
    a.dim_num = len(shape)
    for i, s in enumerate(shape):
        a.dims[i] = s
    if host is not None:
        a.host_data = host.ctypes.data
    a._keep_alive = (t, host)   # the record holds raw addresses: keep the arrays they point into alive with it
    return a


class Context:
    def __init__(self, stream_ptr=None):
        self.handle = ctypes.c_void_p()
        _check(lib().atb_b200_context_create(ctypes.byref(self.handle)), "atb_b200_context_create")
        if stream_ptr is not None:
            self.set_stream(stream_ptr)

    def set_stream(self, stream_ptr):
        _check(lib().atb_b200_context_set_stream(self.handle, stream_ptr), "atb_b200_context_set_stream")

    def set_gather(self, peers):
        """Sharded heads: the PaPeers of the next PagedAttention Execute on this context (None switches it off)."""
        _check(lib().atb_b200_context_set_gather(self.handle, None if peers is None else ctypes.byref(peers)),
               "atb_b200_context_set_gather")

    def __del__(self):
        try:
            if self.handle:
                lib().atb_b200_context_destroy(self.handle)
        except Exception:
            pass


class Operation:
    """atb::Operation behind the C wrappers: create from a param struct, then setup() / execute()."""

    def __init__(self, param):
        self.handle = ctypes.c_void_p()
        if isinstance(param, PagedAttentionParam):
            fn, what = lib().atb_b200_operation_create_paged_attention, "CreateOperation(PagedAttentionParam)"
        elif isinstance(param, ReshapeAndCacheWithStrideParam):
            fn, what = (lib().atb_b200_operation_create_reshape_and_cache_with_stride,
                        "CreateOperation(ReshapeAndCacheWithStrideParam)")
        elif isinstance(param, KvCacheParam):
            fn, what = lib().atb_b200_operation_create_kv_cache, "CreateOperation(KvCacheParam)"
        elif isinstance(param, MultiLatentAttentionParam):
            fn, what = (lib().atb_b200_operation_create_multi_latent_attention,
                        "CreateOperation(MultiLatentAttentionParam)")
        elif isinstance(param, NormRopeReshapeParam):
            fn, what = lib().atb_b200_operation_create_norm_rope_reshape, "CreateOperation(NormRopeReshapeParam)"
        elif isinstance(param, BlockCopyParam):
            fn, what = lib().atb_b200_operation_create_block_copy, "CreateOperation(BlockCopyParam)"
        elif isinstance(param, PagedCacheLoadParam):
            fn, what = lib().atb_b200_operation_create_paged_cache_load, "CreateOperation(PagedCacheLoadParam)"
        else:
            fn, what = lib().atb_b200_operation_create_reshape_and_cache, "CreateOperation(ReshapeAndCacheParam)"
        _check(fn(ctypes.byref(param), ctypes.sizeof(param), ctypes.byref(self.handle)), what)

    @property
    def input_num(self):
        n = ctypes.c_uint32()
        _check(lib().atb_b200_operation_input_num(self.handle, ctypes.byref(n)), "GetInputNum")
        return n.value

    @property
    def output_num(self):
        n = ctypes.c_uint32()
        _check(lib().atb_b200_operation_output_num(self.handle, ctypes.byref(n)), "GetOutputNum")
        return n.value

    @property
    def name(self):
        buf = ctypes.create_string_buffer(128)
        _check(lib().atb_b200_operation_name(self.handle, buf, len(buf)), "GetName")
        return buf.value.decode()

    @staticmethod
    def _arr(tensors):
        arr = (AtbTensor * max(len(tensors), 1))()
        for i, t in enumerate(tensors):
            arr[i] = t
        return arr

    def infer_shape(self, ins, n_out):
        outs = (AtbTensor * n_out)()
        _check(lib().atb_b200_operation_infer_shape(self.handle, self._arr(ins), len(ins), outs, n_out), "InferShape")
        return [tuple(outs[i].dims[k] for k in range(outs[i].dim_num)) for i in range(n_out)]

    def setup(self, ins, outs, ctx):
        ws = ctypes.c_uint64(0)
        _check(lib().atb_b200_operation_setup(self.handle, self._arr(ins), len(ins), self._arr(outs), len(outs),
                                              ctypes.byref(ws), ctx.handle if ctx is not None else None), "Setup")
        return ws.value

    def execute(self, ins, outs, workspace_ptr, workspace_bytes, ctx):
        _check(lib().atb_b200_operation_execute(self.handle, self._arr(ins), len(ins), self._arr(outs), len(outs),
                                                workspace_ptr, workspace_bytes,
                                                ctx.handle if ctx is not None else None), "Execute")

    def __del__(self):
        try:
            if self.handle:
                lib().atb_b200_operation_destroy(self.handle)
        except Exception:
            pass
