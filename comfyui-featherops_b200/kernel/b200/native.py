"""ctypes binding of libfeather_b200.so, the C-ABI library declared in include/feather_b200.h.

This is the only place the Python side touches native code.  PyTorch is used for device memory and streams only:
every call passes raw device pointers and the current CUDA stream of the tensors' device.  There is no CPU or
PyTorch fallback: if the library is missing, or a tensor is not on a CUDA device, the call raises.

Stands in for kernel/hip/utils.py:67-129 (`load_hip_stable_extension`) of the reference, which JIT-builds and
loads the HIP extension.
"""

import ctypes
import os
import threading

import torch

_PKG_DIR = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LIB_PATH = os.path.join(_PKG_DIR, "libfeather_b200.so")

FEATHER_OK = 0
FEATHER_ERR_DEVICE_TIMEOUT = 5
OUT_FP16, OUT_BF16 = 0, 1
SRC_FP32, SRC_BF16, SRC_FP16 = 0, 1, 2

_SRC_CODE = {torch.float32: SRC_FP32, torch.bfloat16: SRC_BF16, torch.float16: SRC_FP16}
_OUT_CODE = {torch.float16: OUT_FP16, torch.bfloat16: OUT_BF16}

EXPORTED_SYMBOLS = (
    "launch_scaled_mm",
    "feather_scaled_mm_ex",
    "feather_scaled_mm_workspace_bytes",
    "feather_scaled_mm_choose",
    "feather_scaled_mm_static",
    "feather_scaled_mm_typed",
    "feather_scaled_mm_lora",
    "feather_scaled_mm_multi",
    "feather_scaled_mm_scatter",
    "feather_reduce_partials",
    "feather_copy_block",
    "feather_scaled_mm_static_scratch_bytes",
    "feather_quantize_prepack",
    "feather_prepack_bytes",
    "feather_unprepack_bytes",
    "feather_dequantize",
    "feather_bf16_to_fp16",
    "feather_last_error_string",
    "feather_version",
)


class MMVariant(ctypes.Structure):
    """Mirror of `feather_mm_variant`; all-zero means "library chooses"."""

    _fields_ = [
        ("tokens_tile", ctypes.c_int),
        ("cta_pair", ctypes.c_int),
        ("split_k", ctypes.c_int),
        ("transform_groups", ctypes.c_int),
        ("max_ctas", ctypes.c_int),
        ("kernel", ctypes.c_int),
        ("staging", ctypes.c_int),
    ]

    def as_tuple(self):
        return (self.tokens_tile, self.cta_pair, self.split_k, self.transform_groups, self.max_ctas, self.kernel, self.staging)


class FeatherNativeError(RuntimeError):
    pass


_lib = None
_lib_lock = threading.Lock()


def load_library():
    """Load (once) and return the ctypes handle.  Raises if the library has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lib_lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise FeatherNativeError(
                f"{LIB_PATH} is missing. Build it with `python {os.path.join(_PKG_DIR, 'build.py')}` "
                "(needs nvcc; there is no fallback implementation)."
            )
        lib = ctypes.CDLL(LIB_PATH)
        vp, i64, ci, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
        lib.launch_scaled_mm.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, ci, ci, ci, ci, ci, ci, ci, ci, ci, vp]
        lib.launch_scaled_mm.restype = ci
        lib.feather_scaled_mm_ex.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, ci, ctypes.POINTER(MMVariant), vp, sz, vp, vp]
        lib.feather_scaled_mm_ex.restype = ci
        lib.feather_scaled_mm_workspace_bytes.argtypes = [i64, i64, i64, ctypes.POINTER(MMVariant)]
        lib.feather_scaled_mm_workspace_bytes.restype = sz
        lib.feather_scaled_mm_choose.argtypes = [i64, i64, i64, sz, ctypes.POINTER(MMVariant)]
        lib.feather_scaled_mm_choose.restype = ci
        lib.feather_scaled_mm_static.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, ci, ctypes.POINTER(MMVariant), vp, vp]
        lib.feather_scaled_mm_static.restype = ci
        lib.feather_scaled_mm_multi.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, i64, i64, i64, i64, ci, ctypes.POINTER(MMVariant), vp, vp]
        lib.feather_scaled_mm_multi.restype = ci
        lib.feather_scaled_mm_typed.argtypes = [vp, ci, vp, ci, vp, vp, vp, i64, i64, i64, i64, ci, ci, ctypes.POINTER(MMVariant), vp, sz, vp, vp]
        lib.feather_scaled_mm_typed.restype = ci
        lib.feather_scaled_mm_lora.argtypes = [vp, ci, vp, vp, vp, vp, i64, i64, i64, i64, ci, ci, vp, vp, i64, ctypes.POINTER(MMVariant), vp, vp]
        lib.feather_scaled_mm_lora.restype = ci
        lib.feather_scaled_mm_scatter.argtypes = [vp, vp, vp, vp, ctypes.POINTER(vp), ci, i64, i64, i64, i64, i64, ci, ctypes.POINTER(MMVariant), vp, vp]
        lib.feather_scaled_mm_scatter.restype = ci
        lib.feather_reduce_partials.argtypes = [vp, ci, i64, i64, vp, vp, i64, ctypes.POINTER(vp), ci, i64, ci, vp]
        lib.feather_reduce_partials.restype = ci
        lib.feather_copy_block.argtypes = [vp, i64, vp, i64, i64, i64, vp]
        lib.feather_copy_block.restype = ci
        lib.feather_scaled_mm_static_scratch_bytes.argtypes = []
        lib.feather_scaled_mm_static_scratch_bytes.restype = sz
        lib.feather_quantize_prepack.argtypes = [vp, ci, vp, i64, i64, ci, vp, vp, vp, vp]
        lib.feather_quantize_prepack.restype = ci
        lib.feather_prepack_bytes.argtypes = [vp, i64, i64, ci, vp, vp]
        lib.feather_prepack_bytes.restype = ci
        lib.feather_unprepack_bytes.argtypes = [vp, i64, i64, vp, vp]
        lib.feather_unprepack_bytes.restype = ci
        lib.feather_dequantize.argtypes = [vp, vp, i64, i64, ci, vp, vp]
        lib.feather_dequantize.restype = ci
        lib.feather_bf16_to_fp16.argtypes = [vp, vp, i64, vp]
        lib.feather_bf16_to_fp16.restype = ci
        lib.feather_last_error_string.argtypes = []
        lib.feather_last_error_string.restype = ctypes.c_char_p
        lib.feather_version.argtypes = []
        lib.feather_version.restype = ci
        _lib = lib
    return _lib


def _check(status, what):
    if status != FEATHER_OK:
        msg = load_library().feather_last_error_string().decode("utf-8", "replace")
        raise FeatherNativeError(f"{what} failed (status {status}): {msg}")


def _require_cuda(*tensors):
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise FeatherNativeError("FeatherOps B200 kernels need CUDA tensors; there is no CPU path")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise FeatherNativeError("all tensors must be on the same CUDA device")
    return dev


def _stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


# ------------------------------------------------------------------------------------------------
# Hot-path helpers.  A small-M GEMM runs 15-25 us on the GPU; the general-purpose route (a device context manager, a
# Stream object, seven c_void_p objects per call) measured 19 us of host time per call, so the GEMM entry points use
# the raw-integer forms below.
# ------------------------------------------------------------------------------------------------
try:
    _raw_stream = torch._C._cuda_getCurrentRawStream          # (device index) -> cudaStream_t as int
except AttributeError:                                        # pragma: no cover - older/newer torch without the private hook
    def _raw_stream(index):
        return torch.cuda.current_stream(index).cuda_stream


class _OnDevice:
    """`with _OnDevice(index):` makes `index` the current CUDA device for the C call, and costs nothing when it already is."""

    __slots__ = ("index", "prev")

    def __init__(self, index):
        self.index = index
        self.prev = -1

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc):
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)
        return False


_scratch_ptrs = {}
# torch hands out its side streams from a fixed pool per device, so the number of distinct streams is bounded; a stream beyond
# this many gets no workspace and its GEMMs run without a K split (correct, a little slower at small token counts)
_MAX_STREAM_WORKSPACES = 72


def _scratch_ptrs_for(dev, stream):
    """(device index, workspace pointer, workspace bytes, status-word pointer) for GEMM launches on `stream` (a raw
    cudaStream_t as an int), cached.

    Split-K launches that may overlap on the GPU need separate workspaces (tile counters and fp32 partials live there), so
    the workspace belongs to the (device, stream) pair, not to the device: two threads or side streams doing split-K GEMMs
    on one GPU never share one.  After _MAX_STREAM_WORKSPACES distinct streams a further stream gets no workspace, which
    makes the library choose a variant without a K split for it.  The first stream of a device gets _WORKSPACE_BYTES, every
    further one a quarter of that (the library fits its K split to what it is given).
    """
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    key = (index, stream)
    got = _scratch_ptrs.get(key)
    if got is None:
        st = status_word_for(dev)
        with _scratch_lock:
            n_ws = sum(1 for k in _workspaces if k[1] == index)
        if n_ws < _MAX_STREAM_WORKSPACES:
            ws = workspace_for(dev, stream, nbytes=_WORKSPACE_BYTES if n_ws == 0 else _WORKSPACE_BYTES // 4)
            got = (index, ws.data_ptr(), ws.numel(), st.data_ptr())
        else:
            got = (index, None, 0, st.data_ptr())
        _scratch_ptrs[key] = got
    return got


def _addr(t):
    return t.data_ptr() if t is not None else None


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


# ------------------------------------------------------------------------------------------------
# Per-device scratch owned by the Python side (the C ABI never allocates).
# ------------------------------------------------------------------------------------------------
_WORKSPACE_BYTES = 64 << 20   # split-K partials; covers every shape in the shipped heuristics
_scratch_lock = threading.Lock()
_workspaces = {}
_status_words = {}
_amax_words = {}


def workspace_for(device, stream=None, nbytes=None):
    """Zero-initialised split-K workspace for launches on `stream` of `device` (a raw cudaStream_t as an int; default: the
    current stream), allocated on first use through torch's allocator.

    The kernel leaves the tile counters at the start of the workspace at zero after every launch, so one buffer
    serves every later call on the same stream; launches on another stream get a buffer of their own.
    """
    index = device.index if device.index is not None else torch.cuda.current_device()
    if stream is None:
        stream = _raw_stream(index)
    key = (device.type, index, stream)
    with _scratch_lock:
        ws = _workspaces.get(key)
        if ws is None:
            ws = torch.zeros(_WORKSPACE_BYTES if nbytes is None else nbytes, dtype=torch.uint8, device=device)
            # the zero fill ran on torch's current stream; the first GEMM may be enqueued on another one
            torch.cuda.current_stream(device).synchronize()
            _workspaces[key] = ws
        return ws


def status_word_for(device):
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    with _scratch_lock:
        st = _status_words.get(key)
        if st is None:
            # word 0: status; words 2.. : 32 int64 cycle counters filled when FEATHER_STATS is set (profiling aid)
            st = torch.zeros(2 + 64, dtype=torch.int32, device=device)
            _status_words[key] = st
        return st


def _amax_word_for(device):
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    with _scratch_lock:
        w = _amax_words.get(key)
        if w is None:
            w = torch.zeros(2, dtype=torch.int32, device=device)
            _amax_words[key] = w
        return w


def check_device_status(device=None):
    """Synchronise `device` and raise if a kernel recorded a failure (a bounded wait that ran out).

    The hot path never calls this (it would serialise the stream); tests and debugging do.
    """
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    st = status_word_for(device)
    value = int(st[0].item())
    if value != 0:
        st.zero_()
        # a launch that gave up may have left split-K tile counters behind: every later split-K launch on that workspace
        # would reduce too early or never, so put the counters of this device's workspaces back to zero
        index = device.index if device.index is not None else torch.cuda.current_device()
        with _scratch_lock:
            for key, ws in _workspaces.items():
                if key[1] == index:
                    ws[:65536].zero_()
        torch.cuda.synchronize(device)
        role = (value >> 8) & 0xFF
        detail = (value >> 16) & 0xFFFF
        names = {1: "TMA producer", 2: "MMA issuer", 3: "transform warp", 4: "epilogue warp"}
        raise FeatherNativeError(
            f"scaled_mm kernel reported status {value & 0xFF} ({names.get(role, 'role ' + str(role))}, detail 0x{detail:x}): "
            "a bounded wait ran out and the kernel returned early; the output is not valid"
        )


def read_stats(device):
    """Cycle counters of CTA 0 from the last scaled_mm launch made with FEATHER_STATS=1 in the environment."""
    torch.cuda.synchronize(device)
    v = status_word_for(device)[2:66].view(torch.int64).cpu().tolist()
    return {
        "raw": v,
        "producer": {"total": v[0], "wait_stage_free": v[1]},
        "w_producer": {"total": v[2], "wait_stage_free": v[3]},
        "mma": {"total": v[4], "wait_acc_free": v[5], "wait_tokens": v[6], "wait_weights": v[7]},
        "mma_detail": {"tok_head": v[16], "wgt_head": v[17], "tok_events": v[18], "wgt_events": v[19], "tok_max": v[20], "wgt_max": v[21], "kblocks": v[22], "issue": v[23]},
        "transform": {"total": v[8], "wait_weight_bytes": v[9], "wait_tmem_free": v[10]},
        "epilogue": {"total": v[12], "wait_acc_full": v[13], "store_chunks": v[14], "chunks": v[15]},
    }


# ------------------------------------------------------------------------------------------------
# GEMM
# ------------------------------------------------------------------------------------------------
KERNEL_AUTO, KERNEL_TMEM, KERNEL_STREAM = 0, 1, 2


def make_variant(tokens_tile=0, cta_pair=0, split_k=0, transform_groups=0, max_ctas=0, kernel=0, staging=0):
    return MMVariant(tokens_tile, cta_pair, split_k, transform_groups, max_ctas, kernel, staging)


def choose_variant(M, N, K, workspace_bytes=_WORKSPACE_BYTES):
    v = MMVariant()
    _check(load_library().feather_scaled_mm_choose(M, N, K, workspace_bytes, ctypes.byref(v)), "feather_scaled_mm_choose")
    return v


def workspace_bytes(M, N, K, variant=None):
    return int(load_library().feather_scaled_mm_workspace_bytes(M, N, K, ctypes.byref(variant) if variant is not None else None))


def scaled_mm_into(a, b_prepacked, scale, bias, c, variant=None, n_cols=None):
    """c[:, :N] = cvt((a @ up(b)) * scale) + bias on the current stream of a's device.  No allocation, no sync.

    `c` may be a column slice of a wider row-major buffer (stride(0) >= N, stride(1) == 1): that is how a weight
    shard writes its block of columns in place.
    """
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale, bias, c)
    M, K = a.shape
    N = b_prepacked.shape[1] if n_cols is None else n_cols
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = _raw_stream(index)
    index, ws_ptr, ws_bytes, st_ptr = _scratch_ptrs_for(dev, stream)
    with _OnDevice(index):
        status = lib.feather_scaled_mm_ex(
            a.data_ptr(), b_prepacked.data_ptr(), _addr(scale), _addr(bias), c.data_ptr(),
            M, N, K, c.stride(0), _OUT_CODE[c.dtype],
            ctypes.byref(variant) if variant is not None else None,
            ws_ptr, ws_bytes, st_ptr, stream,
        )
    if status != FEATHER_OK:
        _check(status, "feather_scaled_mm_ex")
    return c


B_E4M3, B_E5M2 = 0, 1
_B_CODE = {torch.float8_e4m3fn: B_E4M3, torch.float8_e5m2: B_E5M2}


def scaled_mm_typed_into(a, b_prepacked, scale, bias, c, out_dtype=None, variant=None):
    """c = cast_to_c_dtype(cvt_out_dtype((a @ up(b)) * scale) + bias) through `feather_scaled_mm_typed`.

    a: fp16 or bf16 (bf16 is multiplied as it is, no cast pass); b_prepacked: float8_e5m2 or float8_e4m3fn [K/16, N, 16];
    out_dtype: dtype of the rounding and of the bias (default: c's); c may have the other 16-bit dtype, which costs one more
    rounding in the epilogue instead of a separate `y.to(dtype)` pass.
    """
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale, bias, c)
    M, K = a.shape
    N = b_prepacked.shape[1]
    out_dtype = c.dtype if out_dtype is None else out_dtype
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    stream = _raw_stream(index)
    index, ws_ptr, ws_bytes, st_ptr = _scratch_ptrs_for(dev, stream)
    with _OnDevice(index):
        status = lib.feather_scaled_mm_typed(
            a.data_ptr(), _SRC_CODE[a.dtype], b_prepacked.data_ptr(), _B_CODE[b_prepacked.dtype], _addr(scale), _addr(bias), c.data_ptr(),
            M, N, K, c.stride(0), _OUT_CODE[out_dtype], _OUT_CODE[c.dtype],
            ctypes.byref(variant) if variant is not None else None, ws_ptr, ws_bytes, st_ptr, stream,
        )
    if status != FEATHER_OK:
        _check(status, "feather_scaled_mm_typed")
    return c


def scaled_mm_lora_into(a, b_prepacked, scale, bias, c, t, lb_prepacked, out_dtype=None, variant=None):
    """c = cast(cvt((a @ up(b) + t @ lb^T) * scale) + bias): the linear with an un-merged LoRA term folded into the accumulator.
    t [M, R] and lb_prepacked [R/8, N, 8] are fp16 (whatever a's dtype), R a multiple of 64; see `feather_scaled_mm_lora`."""
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale, bias, c, t, lb_prepacked)
    M, K = a.shape
    N = b_prepacked.shape[1]
    R = t.shape[1]
    if t.shape != (M, R) or lb_prepacked.shape != (R // 8, N, 8) or t.dtype != torch.float16 or lb_prepacked.dtype != torch.float16:
        raise FeatherNativeError("LoRA term: t must be [M, R] and lb_prepacked [R/8, N, 8], both float16")
    if not (t.is_contiguous() and lb_prepacked.is_contiguous()):
        raise FeatherNativeError("LoRA term: t and lb_prepacked must be contiguous")
    out_dtype = c.dtype if out_dtype is None else out_dtype
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    st = status_word_for(dev)
    with _OnDevice(index):
        status = lib.feather_scaled_mm_lora(
            a.data_ptr(), _SRC_CODE[a.dtype], b_prepacked.data_ptr(), _addr(scale), _addr(bias), c.data_ptr(), M, N, K, c.stride(0),
            _OUT_CODE[out_dtype], _OUT_CODE[c.dtype], t.data_ptr(), lb_prepacked.data_ptr(), R,
            ctypes.byref(variant) if variant is not None else None, st.data_ptr(), _raw_stream(index),
        )
    if status != FEATHER_OK:
        _check(status, "feather_scaled_mm_lora")
    return c


def scaled_mm_multi_into(a, b_prepacked, scale, bias, outputs, variant=None):
    """One GEMM launch whose epilogue stores every output block to each tensor of `outputs` (same shape/strides; the first is on
    a's device, the others may alias peer GPUs' memory).  Used by the column-sharded linear to fuse the exchange into the GEMM."""
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale, bias, outputs[0])
    M, K = a.shape
    N = b_prepacked.shape[1]
    c0 = outputs[0]
    for c in outputs:
        if c.shape != c0.shape or c.stride() != c0.stride() or c.dtype != c0.dtype:
            raise FeatherNativeError("all output buffers must have the same shape, strides and dtype")
    ptrs = (ctypes.c_void_p * len(outputs))(*[c.data_ptr() for c in outputs])
    st = status_word_for(dev)
    with torch.cuda.device(dev):
        status = lib.feather_scaled_mm_multi(
            _ptr(a), _ptr(b_prepacked), _ptr(scale), _ptr(bias), ptrs, len(outputs), M, N, K, c0.stride(0), _OUT_CODE[c0.dtype],
            ctypes.byref(variant) if variant is not None else None, _ptr(st), _stream_ptr(dev),
        )
    _check(status, "feather_scaled_mm_multi")
    return outputs[0]


def scaled_mm_scatter_into(a, b_prepacked, scale, outputs, rows_per_dst, variant=None):
    """Row-parallel GEMM: this rank's partial of token rows [d*rows_per_dst, (d+1)*rows_per_dst) is stored to outputs[d]
    ([rows_per_dst, N] each, own memory or a peer's).  No bias here: it is added once, by reduce_partials_into."""
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale)
    M, K = a.shape
    N = b_prepacked.shape[1]
    c0 = outputs[0]
    for c in outputs:
        if c.shape != c0.shape or c.stride() != c0.stride() or c.dtype != c0.dtype or c.shape[0] != rows_per_dst:
            raise FeatherNativeError("all row-sharded output buffers must be [rows_per_dst, N] with the same strides and dtype")
    ptrs = (ctypes.c_void_p * len(outputs))(*[c.data_ptr() for c in outputs])
    st = status_word_for(dev)
    with torch.cuda.device(dev):
        status = lib.feather_scaled_mm_scatter(
            _ptr(a), _ptr(b_prepacked), _ptr(scale), None, ptrs, len(outputs), rows_per_dst, M, N, K, c0.stride(0), _OUT_CODE[c0.dtype],
            ctypes.byref(variant) if variant is not None else None, _ptr(st), _stream_ptr(dev),
        )
    _check(status, "feather_scaled_mm_scatter")


def reduce_partials_into(partials, bias, residual, outputs):
    """outputs[d][r, :] = cvt(sum_s fp32(partials[s, r, :])) + bias (+ residual[r, :]) for every destination d.
    partials [n_src, rows, N] on the current device; outputs are [rows, N] views (own memory or peers')."""
    lib = load_library()
    dev = _require_cuda(partials, bias, residual)
    n_src, rows, N = partials.shape
    if not partials.is_contiguous():
        raise FeatherNativeError("partials must be contiguous")
    o0 = outputs[0]
    for o in outputs:
        if o.shape != (rows, N) or o.stride() != o0.stride() or o.dtype != partials.dtype:
            raise FeatherNativeError("every destination must be a [rows, N] view with the partials' dtype and equal strides")
    ptrs = (ctypes.c_void_p * len(outputs))(*[o.data_ptr() for o in outputs])
    with torch.cuda.device(dev):
        status = lib.feather_reduce_partials(
            _ptr(partials), n_src, rows, N, _ptr(bias), _ptr(residual), residual.stride(0) if residual is not None else 0,
            ptrs, len(outputs), o0.stride(0), _OUT_CODE[partials.dtype], _stream_ptr(dev),
        )
    _check(status, "feather_reduce_partials")


def copy_block_into(dst, src, stream=None):
    """dst[:, :] = src[:, :] by a copy engine (`feather_copy_block`), asynchronous on `stream` (default: the current stream).
    Both are 2-D views with unit column stride and the same shape and dtype, on this device or peer-mapped."""
    lib = load_library()
    dev = _require_cuda(src)
    if dst.shape != src.shape or dst.dtype != src.dtype or dst.dim() != 2 or dst.stride(1) != 1 or src.stride(1) != 1:
        raise FeatherNativeError("copy_block_into needs two 2-D views of one shape and dtype with unit column stride")
    item = src.element_size()
    raw = ctypes.c_void_p(stream.cuda_stream) if stream is not None else _stream_ptr(dev)
    with torch.cuda.device(dev):
        status = lib.feather_copy_block(dst.data_ptr(), dst.stride(0) * item, src.data_ptr(), src.stride(0) * item, src.shape[1] * item, src.shape[0], raw)
    _check(status, "feather_copy_block")


def scaled_mm_static_into(a, b_prepacked, scale, bias, c, variant=None):
    """Same result as scaled_mm_into through `feather_scaled_mm_static`: the entry point for callers that cannot allocate
    device memory, whose split-K scratch is a fixed array inside the library.  Raises FeatherNativeError (status 3) when the
    shape needs more scratch than the array holds."""
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale, bias, c)
    M, K = a.shape
    N = b_prepacked.shape[1]
    st = status_word_for(dev)
    with torch.cuda.device(dev):
        status = lib.feather_scaled_mm_static(
            _ptr(a), _ptr(b_prepacked), _ptr(scale), _ptr(bias), _ptr(c), M, N, K, c.stride(0), _OUT_CODE[c.dtype],
            ctypes.byref(variant) if variant is not None else None, _ptr(st), _stream_ptr(dev),
        )
    _check(status, "feather_scaled_mm_static")
    return c


def static_scratch_bytes():
    return int(load_library().feather_scaled_mm_static_scratch_bytes())


def launch_scaled_mm_reference_abi(a, b_prepacked, scale, bias, c, cfg=(1, 8, 4, 8, 2), b_dtype=1):
    """Calls the entry point that keeps the reference's `launch_scaled_mm` argument order. Returns its int result."""
    lib = load_library()
    dev = _require_cuda(a, b_prepacked, scale, bias, c)
    M, K = a.shape
    N = b_prepacked.shape[1]
    with torch.cuda.device(dev):
        return lib.launch_scaled_mm(
            _ptr(a), _ptr(b_prepacked), _ptr(scale), _ptr(bias), _ptr(c), M, N, K,
            1 if scale is not None else 0, 1 if bias is not None else 0, *cfg, b_dtype, _OUT_CODE[c.dtype], _stream_ptr(dev),
        )


# ------------------------------------------------------------------------------------------------
# Weight format
# ------------------------------------------------------------------------------------------------
def quantize_prepack(src, scale=None, premul=None):
    """src [N,K] fp32/bf16/fp16 (contiguous, CUDA) -> (qdata e5m2 [K/16,N,16], scale fp32 0-dim).

    scale=None recalculates amax/57344 (with the reference's zero and fp16-clamp rules); otherwise `scale` is a
    fp32 CUDA tensor with one element that is used as given.  premul (fp32, one element) multiplies an fp32 source first.
    """
    lib = load_library()
    dev = _require_cuda(src, scale, premul)
    N, K = src.shape
    qdata = torch.empty((K // 16, N, 16), dtype=torch.float8_e5m2, device=dev)
    recalc = scale is None
    scale_io = torch.empty((), dtype=torch.float32, device=dev) if recalc else scale.reshape(()).to(torch.float32).clone()
    with torch.cuda.device(dev):
        status = lib.feather_quantize_prepack(
            _ptr(src), _SRC_CODE[src.dtype], _ptr(premul), N, K, 1 if recalc else 0, _ptr(scale_io), _ptr(_amax_word_for(dev)),
            _ptr(qdata), _stream_ptr(dev),
        )
    _check(status, "feather_quantize_prepack")
    return qdata, scale_io


def prepack_bytes(src, src_is_kn=False):
    """e5m2/uint8 [N,K] (or [K,N] when src_is_kn) -> [K/16,N,16], same dtype."""
    lib = load_library()
    dev = _require_cuda(src)
    if src_is_kn:
        K, N = src.shape
    else:
        N, K = src.shape
    dst = torch.empty((K // 16, N, 16), dtype=src.dtype, device=dev)
    with torch.cuda.device(dev):
        status = lib.feather_prepack_bytes(_ptr(src), N, K, 1 if src_is_kn else 0, _ptr(dst), _stream_ptr(dev))
    _check(status, "feather_prepack_bytes")
    return dst


def unprepack_bytes(src):
    lib = load_library()
    dev = _require_cuda(src)
    kb, N, _ = src.shape
    dst = torch.empty((N, kb * 16), dtype=src.dtype, device=dev)
    with torch.cuda.device(dev):
        status = lib.feather_unprepack_bytes(_ptr(src), N, kb * 16, _ptr(dst), _stream_ptr(dev))
    _check(status, "feather_unprepack_bytes")
    return dst


def dequantize(src_prepacked, scale, dtype):
    lib = load_library()
    dev = _require_cuda(src_prepacked, scale)
    kb, N, _ = src_prepacked.shape
    dst = torch.empty((N, kb * 16), dtype=dtype, device=dev)
    with torch.cuda.device(dev):
        status = lib.feather_dequantize(_ptr(src_prepacked), _ptr(scale), N, kb * 16, _SRC_CODE[dtype], _ptr(dst), _stream_ptr(dev))
    _check(status, "feather_dequantize")
    return dst


def bf16_to_fp16(x):
    lib = load_library()
    dev = _require_cuda(x)
    out = torch.empty_like(x, dtype=torch.float16)
    with torch.cuda.device(dev):
        status = lib.feather_bf16_to_fp16(_ptr(x), _ptr(out), x.numel(), _stream_ptr(dev))
    _check(status, "feather_bf16_to_fp16")
    return out
