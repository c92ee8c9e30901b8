"""Python API of the B200 UltraQuant verify/decode attention, mirroring the reference's
`cuda/uq_cuda.py` (reference cuda/uq_cuda.py:10-66): `ext`, `auto_nsplit`, `uq_decode_cuda`,
`workspace_floats`, plus the append hooks `append_kv` (reference uqmt/vllm_adapter.py:48-59) and
`quantize_on_write` (reference uqmt/quant.py:197-206) and the context-split pair
`uq_decode_partial` / `uq_merge`, which the reference does not have.

Everything goes through the C ABI of libuq_b200.so (include/uq_b200.h) with raw device pointers and
the current CUDA stream; torch only owns the memory.  There is no CPU or eager fallback: if the
library is missing or the device is not CUDA, the call raises.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("UQ_B200_LIB") or os.path.join(_HERE, "libuq_b200.so")   # the override is for developers comparing builds
_lib = None
_ext = None

cudaErrorInvalidValue = 1


class UQParams(ctypes.Structure):
    """ctypes mirror of `struct UQParams` (include/uq_params.h; reference cuda/uq_decode.h:11-30)."""
    _fields_ = [("q", ctypes.c_void_p), ("kc", ctypes.c_void_p), ("ks", ctypes.c_void_p), ("vc", ctypes.c_void_p),
                ("vs", ctypes.c_void_p), ("block_table", ctypes.c_void_p), ("seq_lens", ctypes.c_void_p),
                ("mo", ctypes.c_void_p), ("ml", ctypes.c_void_p), ("out", ctypes.c_void_p),
                ("B", ctypes.c_int), ("K", ctypes.c_int), ("HQ", ctypes.c_int), ("HKV", ctypes.c_int), ("D", ctypes.c_int),
                ("PAGE", ctypes.c_int), ("max_pages", ctypes.c_int), ("nsplit", ctypes.c_int), ("sm_scale", ctypes.c_float),
                ("variant", ctypes.c_int), ("mb", ctypes.c_int), ("fmt", ctypes.c_int), ("k_ts", ctypes.c_float),
                ("v_ts", ctypes.c_float)]


EXPORTS = ("uqb_block_m", "uqb_mo_elems", "uqb_ml_elems", "uqb_workspace_bytes", "uqb_decode_launch", "uqb_decode_launch_ws",
           "uqb_has_sm90", "uqb_append_launch", "uqb_append_ex_launch", "uqb_append_nvfp4_launch", "uqb_append_nvfp4_ex_launch", "uqb_fwht_launch", "uqb_decode_partial_launch", "uqb_tree_decode_launch", "uqb_merge_launch", "uqb_merge_packed_launch", "uqb_last_status",
           "uqb_last_path", "uqb_launch_count", "uqb_debug_events",
           "uqb_decode_launch_static", "uqb_static_scratch_bytes",
           "uqb_peer_bytes", "uqb_peer_alloc", "uqb_peer_open", "uqb_peer_close", "uqb_peer_free", "uqb_decode_partial_push_launch", "uqb_merge_wait_launch",
           "uqb_cache_to_upstream_launch", "uqb_cache_from_upstream_launch")


def lib():
    """The loaded C-ABI library.  Raises if it has not been built (python -m all_quant_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f"{_LIB_PATH} is missing: build it with `python -m all_quant_b200.build` (there is no fallback path)")
        L = ctypes.CDLL(_LIB_PATH)
        vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        pp = ctypes.POINTER(UQParams)
        L.uqb_block_m.argtypes = [i, i, i]
        for n in ("uqb_mo_elems", "uqb_ml_elems", "uqb_workspace_bytes"):
            getattr(L, n).argtypes = [pp]
            getattr(L, n).restype = sz
        L.uqb_decode_launch.argtypes = [pp, i, i, vp]
        L.uqb_decode_launch_ws.argtypes = [pp, vp, i, i, vp]
        L.uqb_append_launch.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, vp]
        L.uqb_append_ex_launch.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, ctypes.c_float, vp]
        L.uqb_fwht_launch.argtypes = [vp, vp, ctypes.c_longlong, i, i, vp]
        L.uqb_append_nvfp4_launch.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, ctypes.c_float, ctypes.c_float, vp]
        L.uqb_append_nvfp4_ex_launch.argtypes = [vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, ctypes.c_float, ctypes.c_float, i, vp]
        L.uqb_decode_partial_launch.argtypes = [pp, vp, vp, vp, vp]
        L.uqb_merge_launch.argtypes = [vp, vp, i, sz, i, vp, vp]
        L.uqb_tree_decode_launch.argtypes = [pp, vp, vp]
        L.uqb_merge_packed_launch.argtypes = [vp, i, sz, i, vp, vp]
        L.uqb_last_status.argtypes = [ctypes.POINTER(ctypes.c_uint32)]
        L.uqb_launch_count.restype = ctypes.c_ulonglong
        L.uqb_debug_events.argtypes = [vp, vp]
        L.uqb_debug_events.restype = None
        L.uqb_decode_launch_static.argtypes = [pp, i, i, vp]
        L.uqb_static_scratch_bytes.restype = sz
        L.uqb_peer_bytes.argtypes = [i, sz, i]
        L.uqb_peer_bytes.restype = sz
        L.uqb_peer_alloc.argtypes = [sz, ctypes.POINTER(vp), ctypes.c_char_p]
        L.uqb_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.uqb_peer_close.argtypes = [vp]
        L.uqb_peer_free.argtypes = [vp]
        L.uqb_decode_partial_push_launch.argtypes = [pp, vp, ctypes.POINTER(vp), i, i, ctypes.c_uint, vp]
        L.uqb_merge_wait_launch.argtypes = [vp, i, ctypes.c_uint, sz, i, vp, ctypes.c_ulonglong, vp]
        L.uqb_cache_to_upstream_launch.argtypes = [vp, vp, vp, vp, vp, ctypes.c_longlong, i, i, i, i, i, vp]
        L.uqb_cache_from_upstream_launch.argtypes = [vp, vp, vp, vp, vp, ctypes.c_longlong, i, i, i, i, vp]
        _lib = L
    return _lib


_SMS = {}


def _sm_count(device):
    """Multiprocessors of `device`, looked up once (the property query is not free and sat in every call)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _SMS.get(idx)
    if n is None:
        n = _SMS[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def _pow2ceil(v):
    return 1 if v <= 1 else 1 << (int(v) - 1).bit_length()


def _block_m(K, HQ, HKV):
    """uq_block_m in Python (reference cuda/uq_decode.cu:398): the hot path of a call does its size arithmetic here instead of
    through three more library calls; tests/test_abi.py holds the two against each other."""
    return max(16, _pow2ceil(K * _pow2ceil(HQ // HKV)))


class _on_device:
    """`with torch.cuda.device(d)` only when d is not already the current device (the context manager costs a call several
    microseconds; a serving loop is on its device already)."""

    def __init__(self, device):
        self.ctx = None if device.index is None or device.index == torch.cuda.current_device() else torch.cuda.device(device)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *a):
        if self.ctx is not None:
            self.ctx.__exit__(*a)


def _check(err, what):
    if err != 0:
        name = {1: "cudaErrorInvalidValue (shape not served / bad argument)"}.get(err, f"cudaError {err}")
        raise RuntimeError(f"{what} failed: {name}")


def _stream(t):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("uq_cuda: tensors must live on a CUDA device (no CPU path in this library)")


def _params(q, kc, ks, vc, vs, bt, sl, nsplit, sm_scale, variant=0, mb=0, fmt=0, k_ts=1.0, v_ts=1.0):
    B, K, HQ, D = q.shape
    p = UQParams()
    p.q, p.kc, p.ks, p.vc, p.vs = q.data_ptr(), kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr()
    p.block_table, p.seq_lens = bt.data_ptr(), sl.data_ptr()
    p.B, p.K, p.HQ, p.D = B, K, HQ, D
    p.HKV, p.PAGE, p.max_pages, p.nsplit = kc.shape[1], kc.shape[2], bt.shape[1], int(nsplit)
    p.sm_scale, p.variant, p.mb, p.fmt, p.k_ts, p.v_ts = float(sm_scale), int(variant), int(mb), int(fmt), float(k_ts), float(v_ts)
    return p


class _Ext:
    """Stand-in for the reference's pybind module `uq_cuda_ext` (reference cuda/uq_ext.cpp:6-37): same
    four functions, same positional arguments, same checks and messages."""

    @staticmethod
    def block_m(K, HQ, HKV):
        return int(lib().uqb_block_m(int(K), int(HQ), int(HKV)))

    @staticmethod
    def has_sm90():
        return 0

    @staticmethod
    def workspace_floats(B, K, HQ, HKV, D, nsplit):
        p = UQParams()
        p.B, p.K, p.HQ, p.HKV, p.D, p.nsplit = int(B), int(K), int(HQ), int(HKV), int(D), int(nsplit)
        return int(lib().uqb_mo_elems(ctypes.byref(p)) + lib().uqb_ml_elems(ctypes.byref(p)))

    @staticmethod
    def decode(q, kc, ks, vc, vs, bt, sl, nsplit, nwarps, stages, variant, mb, sm_scale, mo=None, ml=None, out=None,
               fmt=0, k_ts=1.0, v_ts=1.0):
        if not (q.is_cuda and q.dtype == torch.bfloat16 and q.is_contiguous()):
            raise RuntimeError("q must be contiguous bf16 cuda")
        if bt.dtype != torch.int32 or sl.dtype != torch.int32:
            raise RuntimeError("bt/sl must be int32")
        _need_cuda(kc, ks, vc, vs, bt, sl)
        if int(fmt) in (0, 1):   # the kernels read D/32 (UltraQuant) or D/16 (NVFP4) scale bytes per row: refuse a cache of the other kind
            per_row = q.shape[-1] // (16 if int(fmt) == 1 else 32)
            if ks.shape[-1] != per_row or vs.shape[-1] != per_row:
                raise RuntimeError(f"scale tensors hold {ks.shape[-1]} / {vs.shape[-1]} bytes per row, fmt={int(fmt)} needs {per_row}")
        p = _params(q, kc, ks, vc, vs, bt, sl, nsplit, sm_scale, variant, mb, fmt, k_ts, v_ts)
        L = lib()
        n_ml = p.B * p.HKV * p.nsplit * _block_m(p.K, p.HQ, p.HKV)
        n_mo = n_ml * p.D
        if mo is None:
            mo = torch.empty(n_mo, dtype=torch.float32, device=q.device)
        if ml is None:
            ml = torch.empty(n_ml, dtype=torch.float32, device=q.device)
        if out is None:
            out = torch.empty_like(q)
        if mo.numel() < n_mo or ml.numel() < n_ml:
            raise RuntimeError("scratch too small")
        p.mo, p.ml, p.out = mo.data_ptr(), ml.data_ptr(), out.data_ptr()
        with _on_device(q.device):
            err = L.uqb_decode_launch(ctypes.byref(p), int(nwarps), int(stages), _stream(q))
        if err:
            _check(err, "uq_decode_launch")
        return out


def ext(verbose=False):
    """The op module (reference cuda/uq_cuda.py:10-31 JIT-builds a pybind extension; here it is a thin
    object over the prebuilt C-ABI library)."""
    global _ext
    if _ext is None:
        lib()
        _ext = _Ext()
    return _ext


def auto_nsplit(B, HKV, n_pages, sms, K=1, G=8):
    """Default number of partial slots (reference cuda/uq_cuda.py:34-37): 4 CTAs per SM, at most one per page, at most 128."""
    target = 4 * sms
    want = max(1, target // max(1, B * HKV))
    return max(1, min(want, n_pages, 128))


def workspace_floats(B, K, HQ, HKV, D, nsplit):
    """fp32 element count of the scratch (mo then ml) for uq_decode_cuda(..., workspace=...) (reference cuda/uq_cuda.py:64-66)."""
    return ext().workspace_floats(B, K, HQ, HKV, D, nsplit)


def uq_decode_cuda(q, kc, ks, vc, vs, block_table, seq_lens, *, fused=True, nsplit=None, nwarps=0, stages=0, variant=0, mb=0,
                   sm_scale=None, out=None, fmt=0, k_ts=1.0, v_ts=1.0, workspace=None):
    """Fused K-query verify attention over the paged FP4 cache (reference cuda/uq_cuda.py:40-61).

    q bf16 [B,K,Hq,D]; kc/vc uint8 [pages,Hkv,PAGE,D/2]; ks/vs uint8 [pages,Hkv,PAGE,D/32] (fmt=1, the NVFP4 cache:
    e4m3fn bytes [pages,Hkv,PAGE,D/16] and the per-tensor scales k_ts / v_ts, reference uqmt/nvfp4.py:257-278); block_table
    int [B,max_pages]; seq_lens int [B] including the K draft tokens.  Returns bf16 [B,K,Hq,D].
    fused=False is the reference's no-sharing mode: K independent single-query problems over B*K
    pseudo-sequences (the cache is read K times)."""
    _need_cuda(q, kc, ks, vc, vs, block_table, seq_lens)
    B, K, HQ, D = q.shape
    HKV = kc.shape[1]
    sm_scale = sm_scale if sm_scale is not None else D ** -0.5
    if seq_lens.dtype != torch.int32:
        seq_lens = seq_lens.to(torch.int32)
    if block_table.dtype != torch.int32:
        block_table = block_table.to(torch.int32)
    if not q.is_contiguous():
        q = q.contiguous()
    if nsplit is None:
        nsplit = auto_nsplit(B, HKV, block_table.shape[1], _sm_count(q.device), K, HQ // HKV)
    e = ext()
    mo = ml = None
    if workspace is not None:   # caller-owned fp32 scratch, nothing is allocated inside
        n_ml = B * HKV * int(nsplit) * _block_m(K, HQ, HKV)
        mo = workspace[: n_ml * D]
        ml = workspace[n_ml * D: n_ml * (D + 1)]
    if fused or K == 1:
        return e.decode(q, kc, ks, vc, vs, block_table, seq_lens, nsplit, nwarps, stages, variant, mb, sm_scale, mo, ml, out, fmt, k_ts, v_ts)
    qs = q.reshape(B * K, 1, HQ, D)
    bt = block_table.repeat_interleave(K, 0)
    sl = (seq_lens.repeat_interleave(K) - K + torch.arange(K, device=q.device).repeat(B) + 1).to(torch.int32)
    return e.decode(qs, kc, ks, vc, vs, bt, sl, nsplit, nwarps, stages, variant, mb, sm_scale, None, None, None, fmt, k_ts, v_ts).reshape(B, K, HQ, D)


# ---- tree-masked verify (reference uqmt/tree.py) -------------------------------------------------------------------
def chain_mask(K, B=None, device="cpu"):
    """Bit t of entry j set for t <= j: the ordinary causal verify (reference uqmt/tree.py:27-29)."""
    m = torch.tensor([(1 << (j + 1)) - 1 for j in range(K)], dtype=torch.int32, device=device)
    return m if B is None else m.expand(B, K).contiguous()


def parents_to_mask(parents):
    """parents [..., K] (parents[j] < j, -1 = child of the committed prefix) -> int32 [..., K] ancestor-or-self
    bitmasks (reference uqmt/tree.py:37-47)."""
    p = torch.as_tensor(parents, dtype=torch.int64)
    K = p.shape[-1]
    m = torch.zeros_like(p)
    for j in range(K):
        par = p[..., j]
        pm = torch.where(par >= 0, torch.gather(m, -1, par.clamp_min(0).unsqueeze(-1)).squeeze(-1), torch.zeros_like(par))
        m[..., j] = pm | (1 << j)
    return m.to(torch.int32)


def star_mask(K, device="cpu"):
    """Token 0 is the root draft, tokens 1..K-1 its children (reference uqmt/tree.py:32-34)."""
    return parents_to_mask([-1] + [0] * (K - 1)).to(device)


def uq_tree_decode(q, kc, ks, vc, vs, block_table, seq_lens, tree_mask=None, *, nsplit=None, sm_scale=None, out=None,
                   workspace=None):
    """Fused K-query verify with a per-sequence tree mask (reference uqmt/tree.py:130-166): the K tree tokens are the
    last K cache positions; query j sees the committed prefix and tree token t iff bit t of tree_mask[b, j] is set.
    tree_mask int32 [B,K] or [K] (broadcast), 1 <= K <= 16; None = chain = uq_decode_cuda.  Returns bf16 [B,K,Hq,D]."""
    _need_cuda(q, kc, ks, vc, vs, block_table, seq_lens)
    if q.dim() != 4 or q.dtype != torch.bfloat16:
        raise RuntimeError("q must be bf16 [B,K,Hq,D]")
    B, K, HQ, D = q.shape
    if not 1 <= K <= 16:
        raise RuntimeError("1 <= K <= 16")
    if tree_mask is None:
        return uq_decode_cuda(q, kc, ks, vc, vs, block_table, seq_lens, nsplit=nsplit, sm_scale=sm_scale, out=out, workspace=workspace)
    HKV = kc.shape[1]
    sm_scale = sm_scale if sm_scale is not None else D ** -0.5
    seq_lens = seq_lens.to(torch.int32)
    block_table = block_table.to(torch.int32).contiguous()
    q = q.contiguous()
    tm = tree_mask.to(device=q.device, dtype=torch.int32)
    tm = (tm.expand(B, K) if tm.dim() == 1 else tm).contiguous()
    if nsplit is None:
        nsplit = auto_nsplit(B, HKV, block_table.shape[1], _sm_count(q.device), K, HQ // HKV)
    p = _params(q, kc, ks, vc, vs, block_table, seq_lens, nsplit, sm_scale)
    L = lib()
    n_mo, n_ml = int(L.uqb_mo_elems(ctypes.byref(p))), int(L.uqb_ml_elems(ctypes.byref(p)))
    if workspace is None:
        workspace = torch.empty(n_mo + n_ml, dtype=torch.float32, device=q.device)
    if workspace.numel() < n_mo + n_ml:
        raise RuntimeError("scratch too small")
    if out is None:
        out = torch.empty_like(q)
    p.mo, p.ml, p.out = workspace.data_ptr(), workspace.data_ptr() + 4 * n_mo, out.data_ptr()
    with torch.cuda.device(q.device):
        err = L.uqb_tree_decode_launch(ctypes.byref(p), tm.data_ptr(), _stream(q))
    _check(err, "uq_tree_decode_launch")
    return out


def uq_decode_static(q, kc, ks, vc, vs, block_table, seq_lens, out, *, nsplit=None, sm_scale=None):
    """uq_decode_cuda for hosts that may not allocate device memory around the call: the split-KV partials go to the
    24 MiB array built into the library instead of a torch allocation, and `out` (bf16, shape of q) must be supplied.
    block_table / seq_lens must already be int32 and q contiguous, so that nothing is converted (and allocated) here.
    Raises if the call's partials do not fit the built-in array; calls sharing a device must not overlap on the GPU."""
    _need_cuda(q, kc, ks, vc, vs, block_table, seq_lens, out)
    if not (q.dtype == torch.bfloat16 and q.is_contiguous() and out.dtype == torch.bfloat16 and out.is_contiguous() and out.shape == q.shape):
        raise RuntimeError("q and out must be contiguous bf16 of the same shape")
    if block_table.dtype != torch.int32 or seq_lens.dtype != torch.int32 or not block_table.is_contiguous():
        raise RuntimeError("bt/sl must be int32 (contiguous)")
    B, K, HQ, D = q.shape
    HKV = kc.shape[1]
    if nsplit is None:
        nsplit = auto_nsplit(B, HKV, block_table.shape[1], _sm_count(q.device), K, HQ // HKV)
    p = _params(q, kc, ks, vc, vs, block_table, seq_lens, nsplit, sm_scale if sm_scale is not None else D ** -0.5)
    p.out = out.data_ptr()
    L = lib()
    need, have = int(L.uqb_workspace_bytes(ctypes.byref(p))), int(L.uqb_static_scratch_bytes())
    if need > have:
        raise RuntimeError(f"this call needs {need} bytes of partials, the built-in scratch holds {have}: lower nsplit or pass a workspace to uq_decode_cuda")
    with torch.cuda.device(q.device):
        err = L.uqb_decode_launch_static(ctypes.byref(p), 0, 0, _stream(q))
    _check(err, "uq_decode_launch_static")
    return out


_DTYPE = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


PAPER_C = 0.156   # the constant of the 'paper' scale rule (reference uqmt/quant.py:35)


_KERNEL_FLAG = {None: 0, "bulk": 4, "rows": 8}


def _rule_flags(rule, c, rotate_k=False, kernel=None):
    if rule not in ("ceil", "paper"):
        raise ValueError(rule)
    if kernel not in _KERNEL_FLAG:
        raise ValueError(f"append kernel {kernel!r}: None (by the size of the call), 'bulk' or 'rows'")
    return (1 if rotate_k else 0) | (2 if rule == "paper" else 0) | _KERNEL_FLAG[kernel], float(PAPER_C if c is None else c)


def fwht(x, out=None):
    """Orthonormal Walsh-Hadamard transform along the last axis (reference uqmt/quant.py:84-98), D in {64,128,256}: what the
    queries of a cache with rotated keys go through (rotate_kq, :105-107).  Same dtype out as in; `out` may be `x`."""
    _need_cuda(x)
    if x.dtype not in _DTYPE:
        raise RuntimeError("x must be fp32, bf16 or fp16")
    x = x.contiguous()
    out = torch.empty_like(x) if out is None else out
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise RuntimeError("out must be contiguous with x's shape and dtype")
    D = x.shape[-1]
    with torch.cuda.device(x.device):
        err = lib().uqb_fwht_launch(x.data_ptr(), out.data_ptr(), x.numel() // max(1, D), D, _DTYPE[x.dtype], _stream(x))
    _check(err, "uq_fwht_launch")
    return out


def append_kv(kc, ks, vc, vs, key, value, slot_mapping, *, rotate_k=False, rule="ceil", c=None, kernel=None):
    """Quantize new key/value [T,Hkv,D] and write them at flat slots (slot = physical_page * PAGE + offset):
    the cache-append hook of an engine (reference uqmt/vllm_adapter.py:48-59).  One kernel launch for both streams;
    bytes identical to the reference encoder.  Negative slots are skipped.
    rotate_k: the keys go through the orthonormal Hadamard transform first (feed the verify call fwht(q));
    rule / c: the scale rule of the reference's configurable quantiser (uqmt/quant.py:52-70), 'ceil' or 'paper'.
    kernel: None picks by the size of the call (a prompt's worth of rows goes to the bulk kernel, which runs at memory
    bandwidth; a decode step to the one-warp-per-row kernel), 'bulk' / 'rows' name one (same bytes)."""
    flags, c = _rule_flags(rule, c, rotate_k, kernel)
    _need_cuda(kc, ks, vc, vs, key, value, slot_mapping)
    if key.dtype not in _DTYPE or value.dtype != key.dtype:
        raise RuntimeError("key/value must both be fp32, bf16 or fp16")
    T, HKV, D = key.shape
    key, value = key.contiguous(), value.contiguous()
    slots = slot_mapping.to(torch.int64).contiguous()
    for t in (kc, ks, vc, vs):
        if not t.is_contiguous() or t.dtype != torch.uint8:
            raise RuntimeError("cache tensors must be contiguous uint8")
    with torch.cuda.device(key.device):
        err = lib().uqb_append_ex_launch(kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), key.data_ptr(), value.data_ptr(),
                                         slots.data_ptr(), T, HKV, D, kc.shape[2], _DTYPE[key.dtype], flags, c, _stream(key))
    _check(err, "uq_append_launch")


def append_kv_nvfp4(kc, ks, vc, vs, key, value, slot_mapping, k_ts, v_ts, kernel=None):
    """The append for an NVFP4 cache (fmt=1): key/value [T,Hkv,D] -> e2m1 codes and one e4m3fn scale byte per 16 channels
    (ks/vs [pages,Hkv,PAGE,D/16]) for the per-tensor scales k_ts / v_ts, which the decode call takes as well.  Bytes
    identical to the reference's quantize_nvfp4(x, tensor_scale) (uqmt/quant.py:125-136); one kernel launch (kernel as in
    append_kv: by the size of the call, or 'bulk' / 'rows')."""
    if kernel not in _KERNEL_FLAG:
        raise ValueError(f"append kernel {kernel!r}: None (by the size of the call), 'bulk' or 'rows'")
    _need_cuda(kc, ks, vc, vs, key, value, slot_mapping)
    if key.dtype not in _DTYPE or value.dtype != key.dtype:
        raise RuntimeError("key/value must both be fp32, bf16 or fp16")
    T, HKV, D = key.shape
    if ks.shape[-1] != D // 16 or vs.shape[-1] != D // 16:
        raise RuntimeError(f"an NVFP4 cache has {D // 16} scale bytes per row")
    key, value = key.contiguous(), value.contiguous()
    slots = slot_mapping.to(torch.int64).contiguous()
    for t in (kc, ks, vc, vs):
        if not t.is_contiguous() or t.dtype != torch.uint8:
            raise RuntimeError("cache tensors must be contiguous uint8")
    with torch.cuda.device(key.device):
        err = lib().uqb_append_nvfp4_ex_launch(kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), key.data_ptr(), value.data_ptr(),
                                               slots.data_ptr(), T, HKV, D, kc.shape[2], _DTYPE[key.dtype], float(k_ts), float(v_ts),
                                               _KERNEL_FLAG[kernel], _stream(key))
    _check(err, "uq_append_nvfp4_launch")


def to_upstream_layout(kc, ks, vc, vs, slot_bytes=None, *, canon_negzero=False, zero_sentinel=False, out=None):
    """This library's cache arrays -> the upstream engines' slot array uint8 [pages, PAGE, Hkv, slot_bytes] (slot = K codes, K
    scale bytes, V codes, V scale bytes, zero padding; reference cuda/UPSTREAM_COMPAT.md:81-88).  canon_negzero writes a
    minus-zero code as zero, zero_sentinel gives an all-zero group the scale byte 0: with both, a 'paper'-rule cache carries the
    upstream encoder's bytes (reference cuda/UPSTREAM_COMPAT.md:93-95)."""
    _need_cuda(kc, ks, vc, vs)
    pages, HKV, PAGE, half = kc.shape
    D = 2 * half
    slot_bytes = D + 2 * (D // 32) if slot_bytes is None else int(slot_bytes)
    for t in (kc, ks, vc, vs):
        if not t.is_contiguous() or t.dtype != torch.uint8:
            raise RuntimeError("cache tensors must be contiguous uint8")
    if out is None:
        out = torch.empty(pages, PAGE, HKV, slot_bytes, dtype=torch.uint8, device=kc.device)
    with _on_device(kc.device):
        err = lib().uqb_cache_to_upstream_launch(kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), out.data_ptr(), pages, HKV, PAGE, D, slot_bytes,
                                                 (1 if canon_negzero else 0) | (2 if zero_sentinel else 0), _stream(kc))
    _check(err, "uq_cache_to_upstream_launch")
    return out


def from_upstream_layout(cache, D):
    """The upstream engines' slot array uint8 [pages, PAGE, Hkv, slot >= D + D/16] -> (kc, ks, vc, vs) of this library
    (reference cuda/UPSTREAM_COMPAT.md:81-85); the page table and seq_lens carry over unchanged."""
    _need_cuda(cache)
    if cache.dtype != torch.uint8 or not cache.is_contiguous() or cache.dim() != 4:
        raise RuntimeError("cache must be contiguous uint8 [pages, PAGE, Hkv, slot]")
    pages, PAGE, HKV, slot = cache.shape
    G = D // 32
    kc = torch.empty(pages, HKV, PAGE, D // 2, dtype=torch.uint8, device=cache.device)
    ks = torch.empty(pages, HKV, PAGE, G, dtype=torch.uint8, device=cache.device)
    vc, vs = torch.empty_like(kc), torch.empty_like(ks)
    with _on_device(cache.device):
        err = lib().uqb_cache_from_upstream_launch(cache.data_ptr(), kc.data_ptr(), ks.data_ptr(), vc.data_ptr(), vs.data_ptr(), pages, HKV, PAGE, D, slot, _stream(cache))
    _check(err, "uq_cache_from_upstream_launch")
    return kc, ks, vc, vs


def quantize_on_write(x, code, scale, slots, rule="ceil", c=None, kernel=None):
    """Quantize x [N,Hkv,D] and scatter into `code` [pages,Hkv,PAGE,D/2] / `scale` [pages,Hkv,PAGE,D/32] at flat
    slots [N] (reference uqmt/quant.py:197-206); rule 'ceil' (the cache's own encoder) or 'paper' with constant c;
    kernel as in append_kv."""
    flags, c = _rule_flags(rule, c, kernel=kernel)
    _need_cuda(x, code, scale, slots)
    if x.dtype not in _DTYPE:
        raise RuntimeError("x must be fp32, bf16 or fp16")
    N, HKV, D = x.shape
    x = x.contiguous()
    sl = slots.to(torch.int64).contiguous()
    with torch.cuda.device(x.device):
        err = lib().uqb_append_ex_launch(code.data_ptr(), scale.data_ptr(), None, None, x.data_ptr(), None, sl.data_ptr(),
                                         N, HKV, D, code.shape[2], _DTYPE[x.dtype], flags, c, _stream(x))
    _check(err, "uq_append_launch")


def uq_decode_partial(q, kc, ks, vc, vs, block_table, seq_lens, pos_offset=None, *, nsplit=None, sm_scale=None, workspace=None,
                      into=None):
    """Attention over one context shard (the cache and block_table hold only this shard's pages; shard-local key 0 of
    sequence b is global position pos_offset[b]; seq_lens are global).  Returns (o fp32 [B,K,Hq,D] normalised,
    lse2 fp32 [B,K,Hq] in the log2 domain, -inf for rows that see nothing here).  Not in the reference."""
    _need_cuda(q, kc, ks, vc, vs, block_table, seq_lens, pos_offset)
    B, K, HQ, D = q.shape
    HKV = kc.shape[1]
    sm_scale = sm_scale if sm_scale is not None else D ** -0.5
    seq_lens = seq_lens.to(torch.int32)
    block_table = block_table.to(torch.int32).contiguous()
    q = q.contiguous()
    if nsplit is None:
        nsplit = auto_nsplit(B, HKV, block_table.shape[1], _sm_count(q.device), K, HQ // HKV)
    p = _params(q, kc, ks, vc, vs, block_table, seq_lens, nsplit, sm_scale)
    L = lib()
    n_mo, n_ml = int(L.uqb_mo_elems(ctypes.byref(p))), int(L.uqb_ml_elems(ctypes.byref(p)))
    if workspace is None:
        workspace = torch.empty(n_mo + n_ml, dtype=torch.float32, device=q.device)
    if workspace.numel() < n_mo + n_ml:
        raise RuntimeError("scratch too small")
    p.mo, p.ml = workspace.data_ptr(), workspace.data_ptr() + 4 * n_mo
    if into is not None:   # one packed fp32 buffer of B*K*Hq*(D+1) floats: o, then lse2 (what uq_merge_packed takes)
        n_o = B * K * HQ * D
        o, lse = into[:n_o].view(B, K, HQ, D), into[n_o: n_o + B * K * HQ].view(B, K, HQ)
    else:
        o = torch.empty(B, K, HQ, D, dtype=torch.float32, device=q.device)
        lse = torch.empty(B, K, HQ, dtype=torch.float32, device=q.device)
    po = None if pos_offset is None else pos_offset.to(torch.int32).contiguous()
    with torch.cuda.device(q.device):
        err = L.uqb_decode_partial_launch(ctypes.byref(p), None if po is None else po.data_ptr(), o.data_ptr(), lse.data_ptr(), _stream(q))
    _check(err, "uq_decode_partial_launch")
    return o, lse


def uq_merge(o_parts, lse2_parts, out=None):
    """Merge R shards' partials: o_parts fp32 [R,...,D], lse2_parts fp32 [R,...] -> bf16 [...,D].  Not in the reference."""
    _need_cuda(o_parts, lse2_parts)
    o_parts, lse2_parts = o_parts.contiguous(), lse2_parts.contiguous()
    R, D = o_parts.shape[0], o_parts.shape[-1]
    rows = lse2_parts[0].numel()
    if out is None:
        out = torch.empty(o_parts.shape[1:], dtype=torch.bfloat16, device=o_parts.device)
    with torch.cuda.device(o_parts.device):
        err = lib().uqb_merge_launch(o_parts.data_ptr(), lse2_parts.data_ptr(), R, rows, D, out.data_ptr(), _stream(o_parts))
    _check(err, "uq_merge_launch")
    return out


def uq_merge_packed(packed, rows, D, out):
    """Merge of R shards whose partials are packed buffers (o [rows,D], then lse2 [rows]): packed fp32 [R, rows*(D+1)] ->
    out bf16 [..., D] with rows rows.  Not in the reference."""
    _need_cuda(packed, out)
    packed = packed.contiguous()
    with torch.cuda.device(packed.device):
        err = lib().uqb_merge_packed_launch(packed.data_ptr(), packed.shape[0], rows, D, out.data_ptr(), _stream(packed))
    _check(err, "uq_merge_packed_launch")
    return out


def last_status():
    """(code, block, barrier, tile) of the first device-side wait that ran out since the last call; code 0 = none."""
    a = (ctypes.c_uint32 * 4)()
    _check(lib().uqb_last_status(a), "uq_last_status")
    return tuple(int(v) for v in a)


def last_path():
    """1 = CUDA-core kernel, 2 = tcgen05 kernel (the last decode call of this thread)."""
    return int(lib().uqb_last_path())


def launch_count():
    return int(lib().uqb_launch_count())


# ---------------------------------------------------------------------------------------------- multi-GPU host side
# The reference has no multi-device code.  Two ways to spread the path over the GPUs of one box:
#   (a) KV-head partition: every GPU owns Hkv / N heads of the cache and the matching query heads; no data-path collective.
#   (b) context split: every GPU owns a contiguous range of each sequence's pages; partials are all-gathered and merged.

def head_shard(q, kc, ks, vc, vs, rank, world):
    """Mode (a): this rank's slice of the heads.  Returns contiguous (q [B,K,Hq/N,D], kc, ks, vc, vs [pages,Hkv/N,...]).
    In a deployment each GPU only ever holds its own slice; the page table and seq_lens are the same on every rank."""
    HKV, HQ = kc.shape[1], q.shape[2]
    if HKV % world:
        raise ValueError("the number of KV heads must be divisible by the number of ranks")
    hk, G = HKV // world, HQ // HKV
    sl = slice(rank * hk, (rank + 1) * hk)
    return (q[:, :, rank * hk * G:(rank + 1) * hk * G].contiguous(),) + tuple(t[:, sl].contiguous() for t in (kc, ks, vc, vs))


def context_shard(block_table, rank, world, page_size):
    """Mode (b): this rank's slice of every sequence's page table and the global position of its first key.
    Rank r owns logical pages [r * per, (r + 1) * per) with per = ceil(max_pages / world).  Returns
    (local block_table [B, per], pos_offset int32 [B]); seq_lens stay global."""
    B, max_pages = block_table.shape
    per = max(1, -(-max_pages // world))
    lo, hi = min(rank * per, max_pages), min((rank + 1) * per, max_pages)
    bt = torch.zeros((B, per), dtype=block_table.dtype, device=block_table.device)
    bt[:, : hi - lo] = block_table[:, lo:hi]
    off = torch.full((B,), lo * page_size, dtype=torch.int32, device=block_table.device)
    return bt.contiguous(), off


def uq_decode_context_split(q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset, *, group=None, nsplit=None, sm_scale=None,
                            partial_fn=None, merge_fn=None):
    """Mode (b) on one rank: attention over this rank's context shard, one all-gather of the partials (o fp32 [B,K,Hq,D] and
    lse2 fp32 [B,K,Hq] per rank, packed: K*Hq*(D+1) floats per sequence) over `group`, then the log-sum-exp merge.  Every rank
    returns the full bf16 output.  partial_fn / merge_fn default to the CUDA entry points; the CPU tests of the host logic
    substitute the oracle for them."""
    import torch.distributed as dist
    if partial_fn is None and merge_fn is None:
        # the CUDA path: the partial kernel writes this rank's packed buffer, one all-gather, the merge reads the gathered
        # buffers where they are
        B, K, HQ, D = q.shape
        world = dist.get_world_size(group)
        n = B * K * HQ * (D + 1)
        mine = torch.empty(n, dtype=torch.float32, device=q.device)
        uq_decode_partial(q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset, nsplit=nsplit, sm_scale=sm_scale, into=mine)
        both = torch.empty(world * n, dtype=torch.float32, device=q.device)
        dist.all_gather_into_tensor(both, mine, group=group)
        return uq_merge_packed(both.view(world, n), B * K * HQ, D, torch.empty_like(q))
    partial_fn = partial_fn or uq_decode_partial
    merge_fn = merge_fn or uq_merge
    o, lse = partial_fn(q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset, nsplit=nsplit, sm_scale=sm_scale)
    world = dist.get_world_size(group)
    # one collective instead of two: this rank's partials travel as one flat buffer (o, then lse2)
    n_o, n_l = o.numel(), lse.numel()
    mine = torch.cat([o.reshape(-1), lse.reshape(-1)])
    both = torch.empty(world * (n_o + n_l), dtype=mine.dtype, device=mine.device)
    dist.all_gather_into_tensor(both, mine, group=group)
    both = both.view(world, n_o + n_l)
    o_all = both[:, :n_o].contiguous().view((world,) + tuple(o.shape))
    l_all = both[:, n_o:].contiguous().view((world,) + tuple(lse.shape))
    return merge_fn(o_all, l_all)


class ContextSplit:
    """Mode (b) without a collective call on the data path: every rank owns an exchange buffer that all ranks of the box map
    (CUDA IPC; one process per GPU), a call is two launches per rank - the shard's attention, whose combine kernel stores the
    packed partial into every rank's buffer over NVLink and raises a flag behind it, and the merge, which waits (bounded) for
    all ranks' flags and then merges what has arrived locally.  Not in the reference, which has no multi-GPU code.

    Set-up (allocates and maps memory, exchanges the handles over `group` once): ContextSplit(rows, D, group=...), rows =
    B*K*Hq of the largest call.  Then run(...) per call, the same number of times on every rank.  `wait_ns` bounds the
    merge's wait for the other ranks (0 = one second); a wait that runs out leaves code 3 in last_status() and the output
    of that call undefined - the group should then be abandoned (a rank has left or hangs)."""

    def __init__(self, rows, D, *, group=None, device=None, wait_ns=0, _bases=None, _rank=None):
        L = lib()
        self.rows, self.D, self.wait_ns, self.seq = int(rows), int(D), int(wait_ns), 0
        self._opened, self._own, self._ws = [], None, {}
        if _bases is not None:   # several ranks' objects inside one process (tests on one GPU): the buffers are shared as they are
            self.world, self.rank, self.bases = len(_bases), int(_rank), list(_bases)
            return
        import torch.distributed as dist
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        nbytes = int(L.uqb_peer_bytes(self.world, self.rows, self.D))
        if nbytes == 0:
            raise RuntimeError("ContextSplit: up to 8 ranks")
        own, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
        with torch.cuda.device(dev):
            _check(L.uqb_peer_alloc(nbytes, ctypes.byref(own), handle), "uq_peer_alloc")
            self._own = own.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            self.bases = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.bases.append(self._own)
                    continue
                ptr = ctypes.c_void_p()
                _check(L.uqb_peer_open(h, ctypes.byref(ptr)), "uq_peer_open")
                self._opened.append(ptr.value)
                self.bases.append(ptr.value)
        dist.barrier(group=group)   # nobody stores into a buffer before every rank has mapped all of them

    @staticmethod
    def in_one_process(world, rows, D, wait_ns=0):
        """`world` rank objects that share one process and one GPU (single-GPU tests of the two kernels: their launches run
        one after the other on a stream, none waits for a later one)."""
        L = lib()
        nbytes = int(L.uqb_peer_bytes(world, rows, D))
        bases = []
        for _ in range(world):
            ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            _check(L.uqb_peer_alloc(nbytes, ctypes.byref(ptr), handle), "uq_peer_alloc")
            bases.append(ptr.value)
        objs = [ContextSplit(rows, D, wait_ns=wait_ns, _bases=bases, _rank=r) for r in range(world)]
        objs[0]._owned_all = bases
        return objs

    def push(self, q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset, *, seq, nsplit=None, sm_scale=None):
        """First launch of call `seq`: this rank's shard, its partial stored into every rank's buffer, then the flags."""
        _need_cuda(q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset)
        B, K, HQ, D = q.shape
        if B * K * HQ > self.rows or D != self.D:
            raise RuntimeError("ContextSplit: the call has more rows than the exchange buffers were made for")
        if not (q.is_contiguous() and block_table_local.dtype == torch.int32 and block_table_local.is_contiguous()
                and seq_lens.dtype == torch.int32 and pos_offset.dtype == torch.int32):
            raise RuntimeError("ContextSplit: q contiguous, tables and offsets int32 (nothing is converted on this path)")
        HKV = kc.shape[1]
        if nsplit is None:
            nsplit = auto_nsplit(B, HKV, block_table_local.shape[1], _sm_count(q.device), K, HQ // HKV)
        p = _params(q, kc, ks, vc, vs, block_table_local, seq_lens, nsplit, sm_scale if sm_scale is not None else D ** -0.5)
        L = lib()
        key = (B, K, HQ, HKV, D, int(nsplit), q.device.index)
        ws = self._ws.get(key)
        if ws is None:   # the scratch of this shape: allocated at its first call, kept
            n_mo, n_ml = int(L.uqb_mo_elems(ctypes.byref(p))), int(L.uqb_ml_elems(ctypes.byref(p)))
            ws = self._ws[key] = (torch.empty(n_mo + n_ml, dtype=torch.float32, device=q.device), n_mo)
        p.mo, p.ml = ws[0].data_ptr(), ws[0].data_ptr() + 4 * ws[1]
        bases = (ctypes.c_void_p * self.world)(*self.bases)
        with torch.cuda.device(q.device):
            err = L.uqb_decode_partial_push_launch(ctypes.byref(p), pos_offset.data_ptr(), bases, self.world, self.rank, int(seq), _stream(q))
        _check(err, "uq_decode_partial_push_launch")

    def merge(self, q, out=None, *, seq):
        """Second launch of call `seq`: wait for every rank's flag, merge the slots of the local buffer into `out` (bf16, q's shape)."""
        B, K, HQ, D = q.shape
        out = torch.empty_like(q) if out is None else out
        with torch.cuda.device(q.device):
            err = lib().uqb_merge_wait_launch(self.bases[self.rank], self.world, int(seq), B * K * HQ, D, out.data_ptr(), self.wait_ns, _stream(q))
        _check(err, "uq_merge_wait_launch")
        return out

    def run(self, q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset, *, out=None, nsplit=None, sm_scale=None):
        """One call on this rank: push, then merge.  Every rank returns the full bf16 output."""
        self.seq += 1
        self.push(q, kc, ks, vc, vs, block_table_local, seq_lens, pos_offset, seq=self.seq, nsplit=nsplit, sm_scale=sm_scale)
        return self.merge(q, out, seq=self.seq)

    def close(self):
        """Unmap the other ranks' buffers and free this rank's (after every rank has finished its last call)."""
        L = lib()
        for ptr in self._opened:
            L.uqb_peer_close(ptr)
        self._opened = []
        for ptr in getattr(self, "_owned_all", []):
            L.uqb_peer_free(ptr)
        self._owned_all = []
        if self._own:
            L.uqb_peer_free(self._own)
            self._own = None
