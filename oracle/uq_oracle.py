"""numpy front end of the C oracle (oracle/uq_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this module;
the product package never does.  Each function mirrors one reference CPU function:
  quantize_fp4 / dequantize_fp4   uqmt/attn.py:52-78
  append_kv                       uqmt/vllm_adapter.py:48-59
  reference                       uqmt/attn.py:402-422
Arrays are numpy; bf16 queries are passed as uint16 bit patterns.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force=False):
    """Compile oracle/libuq_oracle.so with gcc (a second or two)."""
    so = os.path.join(_HERE, "libuq_oracle.so")
    src = os.path.join(_HERE, "uq_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "libuq_oracle.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "libuq_oracle.so")
        if not os.path.exists(so):
            build()
        L = ctypes.CDLL(so)
        vp, i32, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
        L.uqo_max_threads.restype = i32
        L.uqo_quantize_fp4.argtypes = [vp, sz, vp, vp]
        L.uqo_dequantize_fp4.argtypes = [vp, vp, sz, vp]
        L.uqo_append_kv.argtypes = [vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]
        L.uqo_reference.argtypes = [vp] * 9 + [i32] * 7 + [f32, vp, vp]
        L.uqo_merge.argtypes = [vp, vp, i32, sz, i32, vp]
        L.uqo_tree_reference.argtypes = [vp] * 8 + [i32] * 7 + [f32, vp]
        L.uqo_quantize_rule.argtypes = [vp, ctypes.c_size_t, i32, f32, vp, vp]
        L.uqo_fwht.argtypes = [vp, ctypes.c_size_t, i32, vp]
        L.uqo_quantize_nvfp4.argtypes = [vp, ctypes.c_size_t, f32, vp, vp]
        L.uqo_e4m3fn_table.argtypes = [vp]
        L.uqo_reference_nvfp4.argtypes = [vp] * 7 + [i32] * 7 + [f32, f32, f32, vp]
        _LIB = L
    return _LIB


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def max_threads():
    return int(lib().uqo_max_threads())


def set_threads(n=0):
    """Threads of the oracle's parallel loops from now on (0 = all processors, whatever OMP_NUM_THREADS said); returns the count."""
    L = lib()
    L.uqo_set_threads.argtypes = [ctypes.c_int]
    L.uqo_set_threads.restype = ctypes.c_int
    return int(L.uqo_set_threads(int(n)))


def bf16_bits(x):
    """fp32 numpy array -> bf16 bit patterns (round to nearest even), as uint16."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(bits):
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def quantize_fp4(x):
    """x [..., D] float -> (packed uint8 [..., D/2], scales uint8 [..., D/32])."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    D = x.shape[-1]
    assert D % 32 == 0, "head_dim must be a multiple of 32"
    packed = np.empty(x.shape[:-1] + (D // 2,), np.uint8)
    scales = np.empty(x.shape[:-1] + (D // 32,), np.uint8)
    lib().uqo_quantize_fp4(_p(x), x.size // 32, _p(packed), _p(scales))
    return packed, scales


def quantize(x, rule="ceil", c=0.156):
    """The configurable quantiser (uqmt/quant.py:63-70): rule 'ceil' = quantize_fp4, 'paper' = round(log2(c * amax))."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    D = x.shape[-1]
    assert D % 32 == 0 and rule in ("ceil", "paper")
    packed = np.empty(x.shape[:-1] + (D // 2,), np.uint8)
    scales = np.empty(x.shape[:-1] + (D // 32,), np.uint8)
    lib().uqo_quantize_rule(_p(x), x.size // 32, 0 if rule == "ceil" else 1, float(c), _p(packed), _p(scales))
    return packed, scales


def fwht(x):
    """Orthonormal Walsh-Hadamard transform along the last axis (uqmt/quant.py:84-98), fp32."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    n = x.shape[-1]
    assert n & (n - 1) == 0
    out = np.empty_like(x)
    lib().uqo_fwht(_p(x), x.size // n, n, _p(out))
    return out


def dequantize_fp4(packed, scales):
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    scales = np.ascontiguousarray(scales, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), np.float32)
    lib().uqo_dequantize_fp4(_p(packed), _p(scales), scales.size, _p(out))
    return out


def append_kv(kc, ks, vc, vs, key, value, slot_mapping):
    """In-place append of key/value [T,Hkv,D] at flat slots (page * PAGE + offset)."""
    for a in (kc, ks, vc, vs):
        assert a.flags["C_CONTIGUOUS"] and a.dtype == np.uint8
    key = np.ascontiguousarray(key, dtype=np.float32)
    value = np.ascontiguousarray(value, dtype=np.float32)
    slots = np.ascontiguousarray(slot_mapping, dtype=np.int64)
    T, HKV, D = key.shape
    lib().uqo_append_kv(_p(kc), _p(ks), _p(vc), _p(vs), _p(key), _p(value), _p(slots), T, HKV, D, kc.shape[2])


def reference(q_bits, kc, ks, vc, vs, block_table, seq_lens, sm_scale=None, pos_offset=None, n_local=None,
              return_lse=False):
    """q_bits uint16 [B,K,Hq,D] (bf16 bit patterns) -> out fp32 [B,K,Hq,D] (and natural-log lse [B,K,Hq])."""
    q_bits = np.ascontiguousarray(q_bits, dtype=np.uint16)
    B, K, HQ, D = q_bits.shape
    _, HKV, PAGE, _ = kc.shape
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    po = None if pos_offset is None else np.ascontiguousarray(pos_offset, dtype=np.int32)
    nl = None if n_local is None else np.ascontiguousarray(n_local, dtype=np.int32)
    kc, ks, vc, vs = (np.ascontiguousarray(a, dtype=np.uint8) for a in (kc, ks, vc, vs))
    out = np.empty((B, K, HQ, D), np.float32)
    lse = np.empty((B, K, HQ), np.float32) if return_lse else None
    sm = float(sm_scale) if sm_scale is not None else D ** -0.5
    lib().uqo_reference(_p(q_bits), _p(kc), _p(ks), _p(vc), _p(vs), _p(bt), _p(sl), _p(po), _p(nl),
                        B, K, HQ, HKV, D, PAGE, bt.shape[1], sm, _p(out), _p(lse))
    return (out, lse) if return_lse else out


def chain_mask(K, B=None):
    """Bit t of entry j set for t <= j: the ordinary causal verify (uqmt/tree.py:27-29)."""
    m = np.array([(1 << (j + 1)) - 1 for j in range(K)], dtype=np.int32)
    return m if B is None else np.ascontiguousarray(np.broadcast_to(m, (B, K)))


def parents_to_mask(parents):
    """parents [..., K] (parents[j] < j, -1 = child of the committed prefix) -> int32 [..., K] ancestor-or-self
    bitmasks (uqmt/tree.py:37-47)."""
    p = np.asarray(parents, dtype=np.int64)
    K = p.shape[-1]
    m = np.zeros_like(p)
    for j in range(K):
        par = p[..., j]
        pm = np.where(par >= 0, np.take_along_axis(m, np.clip(par, 0, None)[..., None], -1)[..., 0], 0)
        m[..., j] = pm | (1 << j)
    return m.astype(np.int32)


def star_mask(K):
    """Token 0 is the root draft, tokens 1..K-1 its children (uqmt/tree.py:32-34)."""
    return parents_to_mask([-1] + [0] * (K - 1))


def tree_reference(q_bits, kc, ks, vc, vs, block_table, seq_lens, tree_mask=None, sm_scale=None):
    """Tree-masked verify (uqmt/tree.py:169-201): tree_mask int32 [B,K] or [K] (broadcast), None = chain."""
    q_bits = np.ascontiguousarray(q_bits, dtype=np.uint16)
    B, K, HQ, D = q_bits.shape
    _, HKV, PAGE, _ = kc.shape
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    tm = None
    if tree_mask is not None:
        tm = np.asarray(tree_mask, dtype=np.int32)
        tm = np.ascontiguousarray(np.broadcast_to(tm, (B, K)))
    kc, ks, vc, vs = (np.ascontiguousarray(a, dtype=np.uint8) for a in (kc, ks, vc, vs))
    out = np.empty((B, K, HQ, D), np.float32)
    sm = float(sm_scale) if sm_scale is not None else D ** -0.5
    lib().uqo_tree_reference(_p(q_bits), _p(kc), _p(ks), _p(vc), _p(vs), _p(bt), _p(sl), _p(tm), B, K, HQ, HKV, D, PAGE,
                             bt.shape[1], sm, _p(out))
    return out


def quantize_nvfp4(x, ts):
    """x [..., D] -> (codes uint8 [..., D/2], e4m3fn scale bytes uint8 [..., D/16]) for the per-tensor scale ts
    (uqmt/quant.py:125-136 with tensor_scale given; uqmt/nvfp4.py:200-203 for the byte view)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    D = x.shape[-1]
    assert D % 16 == 0
    packed = np.empty(x.shape[:-1] + (D // 2,), np.uint8)
    scales = np.empty(x.shape[:-1] + (D // 16,), np.uint8)
    lib().uqo_quantize_nvfp4(_p(x), x.size // 16, float(ts), _p(packed), _p(scales))
    return packed, scales


def e4m3fn_table():
    """fp32 value of every e4m3fn byte (NaN at 0x7f / 0xff)."""
    out = np.empty(256, np.float32)
    lib().uqo_e4m3fn_table(_p(out))
    return out


def reference_nvfp4(q_bits, kc, ks, vc, vs, block_table, seq_lens, k_ts=1.0, v_ts=1.0, sm_scale=None):
    """NVFP4 cache (uqmt/nvfp4.py:257-278): ks / vs are e4m3fn bytes [pages,Hkv,PAGE,D/16], k_ts / v_ts the per-tensor
    fp32 scales.  q_bits uint16 [B,K,Hq,D] -> out fp32 [B,K,Hq,D]."""
    q_bits = np.ascontiguousarray(q_bits, dtype=np.uint16)
    B, K, HQ, D = q_bits.shape
    _, HKV, PAGE, _ = kc.shape
    bt = np.ascontiguousarray(block_table, dtype=np.int32)
    sl = np.ascontiguousarray(seq_lens, dtype=np.int32)
    kc, ks, vc, vs = (np.ascontiguousarray(a, dtype=np.uint8) for a in (kc, ks, vc, vs))
    out = np.empty((B, K, HQ, D), np.float32)
    sm = float(sm_scale) if sm_scale is not None else D ** -0.5
    lib().uqo_reference_nvfp4(_p(q_bits), _p(kc), _p(ks), _p(vc), _p(vs), _p(bt), _p(sl), B, K, HQ, HKV, D, PAGE, bt.shape[1],
                              sm, float(k_ts), float(v_ts), _p(out))
    return out


def merge(o, lse):
    """o [R,rows...,D], lse [R,rows...] (natural log) -> merged [rows...,D]."""
    o = np.ascontiguousarray(o, dtype=np.float32)
    lse = np.ascontiguousarray(lse, dtype=np.float32)
    R, D = o.shape[0], o.shape[-1]
    rows = lse[0].size
    out = np.empty(o.shape[1:], np.float32)
    lib().uqo_merge(_p(o), _p(lse), R, rows, D, _p(out))
    return out


# ---- the upstream engines' slot layout (reference cuda/UPSTREAM_COMPAT.md:81-95, cuda/compat/paper_rule_cpu_check.py:14-18)
def canon_negzero(packed):
    """A code nibble 0x8 (minus zero) becomes 0x0 (the upstream encoder never writes minus zero)."""
    packed = np.asarray(packed, np.uint8)
    lo, hi = packed & 0xF, packed >> 4
    lo = np.where(lo == 8, 0, lo)
    hi = np.where(hi == 8, 0, hi)
    return (lo | (hi << 4)).astype(np.uint8)


def zero_sentinel(packed, scales):
    """Scale byte 0 for every 32-channel group (16 code bytes) whose codes are all zero in magnitude: the upstream encoder's
    mark of an all-zero group."""
    packed, scales = np.asarray(packed, np.uint8), np.asarray(scales, np.uint8).copy()
    groups = packed.reshape(packed.shape[:-1] + (scales.shape[-1], 16))
    scales[((groups & 0x77) == 0).all(-1)] = 0
    return scales


def to_upstream(kc, ks, vc, vs, slot_bytes=None, canon=False, sentinel=False):
    """[pages,Hkv,PAGE,*] x 4 -> uint8 [pages,PAGE,Hkv,slot]: K codes, K scale bytes, V codes, V scale bytes, zero padding."""
    if sentinel:
        ks, vs = zero_sentinel(kc, ks), zero_sentinel(vc, vs)
    if canon:
        kc, vc = canon_negzero(kc), canon_negzero(vc)
    aos = np.concatenate([kc, ks, vc, vs], -1).transpose(0, 2, 1, 3)
    pad = 0 if slot_bytes is None else slot_bytes - aos.shape[-1]
    return np.ascontiguousarray(np.pad(aos, [(0, 0)] * 3 + [(0, pad)]))


def from_upstream(cache, D):
    G = D // 32
    c = np.asarray(cache, np.uint8).transpose(0, 2, 1, 3)
    return tuple(np.ascontiguousarray(a) for a in (c[..., :D // 2], c[..., D // 2:D // 2 + G], c[..., D // 2 + G:D + G], c[..., D + G:D + 2 * G]))
