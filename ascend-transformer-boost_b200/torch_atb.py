"""Python operator API for the decode path, shaped like the reference's `torch_atb` module.

    import torch_atb                                  # here: pkg.torch_atb
    param = torch_atb.PagedAttentionParam(head_num=32, kv_head_num=8, qk_scale=1 / math.sqrt(128))
    op = torch_atb.Operation(param)
    (out,) = op.forward([q, key_cache, value_cache, block_tables, context_lens_cpu])

Mirrors `src/torch_atb/bindings.cpp:49-93, 520-578, 926-945` of the reference (class `Operation` with
`name`, `input_num`, `output_num`, `forward`; `PagedAttentionParam` / `ReshapeAndCacheParam` with
snake_case fields and nested enums; `set_buffer_size`; `Prof`) and the behaviour of
`src/torch_atb/operation_wrapper.cpp:231-319`: `forward` converts the tensors (CPU tensors become
host data, device tensors device data, non-contiguous ones are made contiguous), infers the output
shapes, allocates the outputs, runs Setup and Execute on the library's context and waits for the
stream.  Only the two operations of the decode path exist; graph building is not part of it.

Differences a caller sees: ReshapeAndCache writes its caches in place, so `forward` returns the cache
tensors it was given (the operation rejects outputs that do not alias them); the fields
`mla_v_head_size` and `q_scale` exist here although the reference binding does not expose them.
"""
import enum
import json
import time

from . import capi


class AclDataType(enum.IntEnum):
    ACL_DT_UNDEFINED = -1
    ACL_FLOAT = 0
    ACL_FLOAT16 = 1
    ACL_INT8 = 2
    ACL_INT32 = 3
    ACL_UINT8 = 4
    ACL_INT16 = 6
    ACL_INT64 = 9
    ACL_BOOL = 12
    ACL_BF16 = 27


class InputLayout(enum.IntEnum):
    TYPE_BSND = 0
    TYPE_BNSD = 1


class _Param:
    """Plain attribute bag with the reference binding's keyword constructor and repr."""
    _FIELDS = ()
    _NAME = ""

    def __init__(self, **kw):
        for name, default, _ in self._FIELDS:
            setattr(self, name, default)
        for k, v in kw.items():
            if k not in {f[0] for f in self._FIELDS}:
                raise TypeError(f"{self._NAME}() got an unexpected keyword argument '{k}'")
            setattr(self, k, v)

    def _to_struct(self, struct):
        for name, _, c_name in self._FIELDS:
            v = getattr(self, name)
            setattr(struct, c_name, int(v) if isinstance(v, enum.Enum) else v)
        return struct

    def __repr__(self):
        d = {c_name: (int(getattr(self, name)) if isinstance(getattr(self, name), (enum.Enum, bool)) else
                      getattr(self, name)) for name, _, c_name in self._FIELDS}
        return f"{self._NAME}: " + json.dumps(d)


class PagedAttentionParam(_Param):
    """atb::infer::PagedAttentionParam (include/atb/infer_op_params.h:1859-1963 of the reference)."""
    _NAME = "PagedAttentionParam"

    class MaskType(enum.IntEnum):
        UNDEFINED = 0
        MASK_TYPE_NORM = 1
        MASK_TYPE_ALIBI = 2
        MASK_TYPE_SPEC = 3
        MASK_TYPE_MASK_FREE = 4
        MASK_TYPE_NORM_COMPRESS = 5

    class QuantType(enum.IntEnum):
        TYPE_QUANT_UNQUANT = 0
        TYPE_DEQUANT_FUSION = 1
        TYPE_QUANT_QKV_OFFLINE = 2
        TYPE_QUANT_QKV_ONLINE = 3

    class CompressType(enum.IntEnum):
        COMPRESS_TYPE_UNDEFINED = 0
        COMPRESS_TYPE_KVHEAD = 1
        COMPRESS_TYPE_KVHEAD_ROPE = 2
        COMPRESS_TYPE_MAX = 3

    class CalcType(enum.IntEnum):
        CALC_TYPE_UNDEFINED = 0
        CALC_TYPE_SPEC = 1

    class ScaleType(enum.IntEnum):
        SCALE_TYPE_TOR = 0
        SCALE_TYPE_LOGN = 1
        SCALE_TYPE_MAX = 2

    _FIELDS = (
        ("head_num", 0, "headNum"),
        ("qk_scale", 1.0, "qkScale"),
        ("kv_head_num", 0, "kvHeadNum"),
        ("mask_type", MaskType.UNDEFINED, "maskType"),
        ("batch_run_status_enable", False, "batchRunStatusEnable"),
        ("quant_type", QuantType.TYPE_QUANT_UNQUANT, "quantType"),
        ("out_data_type", AclDataType.ACL_DT_UNDEFINED, "outDataType"),
        ("has_quant_offset", False, "hasQuantOffset"),
        ("compress_type", CompressType.COMPRESS_TYPE_UNDEFINED, "compressType"),
        ("calc_type", CalcType.CALC_TYPE_UNDEFINED, "calcType"),
        ("scale_type", ScaleType.SCALE_TYPE_TOR, "scaleType"),
        ("input_layout", InputLayout.TYPE_BSND, "inputLayout"),
        ("mla_v_head_size", 0, "mlaVHeadSize"),
        ("q_scale", 0.0, "qScale"),
    )

    def _c_param(self):
        return self._to_struct(capi.PagedAttentionParam())


class ReshapeAndCacheParam(_Param):
    """atb::infer::ReshapeAndCacheParam (include/atb/infer_op_params.h:488-530 of the reference)."""
    _NAME = "ReshapeAndCacheParam"

    class CompressType(enum.IntEnum):
        COMPRESS_TYPE_UNDEFINED = 0
        COMPRESS_TYPE_KVHEAD = 1
        COMPRESS_TYPE_KVHEAD_ROPE = 2

    class KvCacheCfg(enum.IntEnum):
        K_CACHE_V_CACHE = 0
        K_CACHE_V_BYPASS = 1

    _FIELDS = (
        ("compress_type", CompressType.COMPRESS_TYPE_UNDEFINED, "compressType"),
        ("kv_cache_cfg", KvCacheCfg.K_CACHE_V_CACHE, "kvCacheCfg"),
    )

    def _c_param(self):
        return self._to_struct(capi.ReshapeAndCacheParam())


# ------------------------------------------------------------------ resources shared by all operations

class _Resources:
    """The library context, a side stream for callers on the legacy default stream, and the workspace
    buffer (src/torch_atb/resource/memory_manager.cpp of the reference keeps one growing buffer too)."""

    def __init__(self):
        self.context = None
        self.side_stream = None
        self.workspace = None
        self.buffer_size = 0

    def stream(self):
        """The operations need an explicit stream (a null stream is rejected, as in the reference): the
        current torch stream when it is not the legacy default one, else a side stream ordered after it."""
        import torch
        cur = torch.cuda.current_stream()
        if cur.cuda_stream != 0:
            return cur, None
        if self.side_stream is None:
            self.side_stream = torch.cuda.Stream()
        self.side_stream.wait_stream(cur)
        return self.side_stream, cur

    def get_context(self, stream):
        if self.context is None:
            self.context = capi.Context()
        self.context.set_stream(stream.cuda_stream)
        return self.context

    def get_workspace(self, nbytes, device):
        import torch
        want = max(int(nbytes), int(self.buffer_size), 256)
        if self.workspace is None or self.workspace.numel() < want or self.workspace.device != device:
            self.workspace = torch.empty(want, dtype=torch.uint8, device=device)
        return self.workspace


_res = _Resources()


def set_buffer_size(bytes):  # noqa: A002  (the reference names the argument `bytes`)
    """Default size of the workspace buffer (grown on demand when an operation needs more)."""
    if bytes < 0:
        raise ValueError("buffer size must not be negative")
    _res.buffer_size = int(bytes)


class Prof:
    """Run-time statistics per operation name (src/torch_atb/prof/prof_stats.cpp of the reference)."""
    _instance = None

    def __init__(self):
        self._run_times = {}

    @staticmethod
    def get_prof_stats():
        if Prof._instance is None:
            Prof._instance = Prof()
        return Prof._instance

    def _set_run_time(self, name, microseconds):
        self._run_times.setdefault(name, []).append(microseconds)

    def get_run_time_stats(self):
        return {k: list(v) for k, v in self._run_times.items()}


# ------------------------------------------------------------------ Operation

def _torch_dtype(code):
    import torch
    return {capi.ACL_FLOAT16: torch.float16, capi.ACL_BF16: torch.bfloat16, capi.ACL_INT8: torch.int8,
            capi.ACL_INT32: torch.int32, capi.ACL_FLOAT: torch.float32, capi.ACL_INT64: torch.int64}[code]


class Operation:
    def __init__(self, param):
        if not isinstance(param, (PagedAttentionParam, ReshapeAndCacheParam)):
            raise TypeError("Operation(): incompatible constructor arguments; supported params are "
                            "PagedAttentionParam and ReshapeAndCacheParam")
        self._param = param
        try:
            self._op = capi.Operation(param._c_param())
        except capi.AtbError as e:
            raise RuntimeError("Failed to create operation") from e
        self._in_place = isinstance(param, ReshapeAndCacheParam)

    @property
    def name(self):
        return self._op.name

    @property
    def input_num(self):
        return self._op.input_num

    @property
    def output_num(self):
        return self._op.output_num

    def __repr__(self):
        return f"op name: {self.name}, input_num: {self.input_num}, output_num: {self.output_num}"

    def forward(self, in_tensors):
        import torch
        t0 = time.perf_counter()
        ins = [t if t.is_contiguous() else t.contiguous() for t in in_tensors]
        device = next((t.device for t in ins if t.is_cuda), None)
        if device is None:
            raise RuntimeError("call Setup fail: no input tensor is on a CUDA device")
        n_out = self.output_num
        a_ins = [capi.atb_tensor(t) for t in ins]
        if self._in_place:
            # key, value, keyCache, valueCache, slotMapping -> keyCache, valueCache
            # key, keyCache, slotMapping -> keyCache                         (K_CACHE_V_BYPASS)
            if len(ins) != self.input_num:
                raise RuntimeError("call operation_->Setup fail")
            outs = [in_tensors[2], in_tensors[3]] if n_out == 2 else [in_tensors[1]]
            if not all(t.is_contiguous() for t in outs):
                raise RuntimeError("call operation_->Setup fail: the caches are written in place and must be contiguous")
        else:
            try:
                shapes = self._op.infer_shape(a_ins, n_out)
            except capi.AtbError as e:
                raise RuntimeError("call operation_->InferShape fail") from e
            out_dtype = ins[0].dtype
            if isinstance(self._param, PagedAttentionParam) and \
                    int(self._param.out_data_type) != int(AclDataType.ACL_DT_UNDEFINED) and ins[0].dtype == torch.int8:
                out_dtype = _torch_dtype(int(self._param.out_data_type))
            outs = [torch.empty(s, dtype=out_dtype, device=device) for s in shapes]
        a_outs = [capi.atb_tensor(t) for t in outs]
        stream, waiter = _res.stream()
        ctx = _res.get_context(stream)
        with torch.cuda.stream(stream):
            try:
                ws_bytes = self._op.setup(a_ins, a_outs, ctx)
            except capi.AtbError as e:
                raise RuntimeError("call operation_->Setup fail") from e
            ws = _res.get_workspace(ws_bytes, device)
            try:
                self._op.execute(a_ins, a_outs, ws.data_ptr(), ws.numel(), ctx)
            except capi.AtbError as e:
                raise RuntimeError("call operation_->Execute fail") from e
        for t in outs:
            t.record_stream(stream)
        stream.synchronize()                      # the reference's forward waits for the stream too
        if waiter is not None:
            waiter.wait_stream(stream)
        Prof.get_prof_stats()._set_run_time(self.name, (time.perf_counter() - t0) * 1e6)
        return outs
