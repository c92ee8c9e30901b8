"""Engine-facing adapter: the varlen inputs of a vLLM-style verify step -> the verify kernel, and the cache-append hook.

Mirror of the reference's uqmt/vllm_adapter.py (same names, arguments and reasons) over this library's CUDA path.
The engine keeps its own block table; the FP4 pool is a side cache indexed by the same physical block ids.
Importing this module needs no GPU; calling uq_verify_attention / append_kv does (there is no CPU path).
"""
import torch

from . import uq_cuda

REASONS = ("ok", "non_uniform_k", "head_dim", "page_size", "q_dtype", "sliding_window", "softcap")
HEAD_DIMS = (64, 128, 256)   # the reference's adapter stops at 128; the kernels here serve 256 as well


def eligible(query, query_start_loc, page_size, *, sliding_window=None, softcap=None):
    """(ok, reason, K) for one step (reference uqmt/vllm_adapter.py:15-34): bf16 queries, a served head_dim, a power-of-two
    page of at least 16 tokens, no sliding window or soft cap, and the same number of query tokens K (1..16) for every
    request.  Reads query_start_loc on the host once: call it in the plan phase of a step, not inside a CUDA graph."""
    if sliding_window not in (None, -1, 0):
        return False, "sliding_window", 0
    if softcap:
        return False, "softcap", 0
    if query.dtype != torch.bfloat16:
        return False, "q_dtype", 0
    if query.shape[-1] not in HEAD_DIMS:
        return False, "head_dim", 0
    if page_size < 16 or page_size & (page_size - 1):
        return False, "page_size", 0
    n = query_start_loc[1:] - query_start_loc[:-1]
    if n.numel() == 0:
        return False, "non_uniform_k", 0
    K = int(n[0])
    if not bool((n == K).all()) or not (1 <= K <= 16):
        return False, "non_uniform_k", 0
    return True, "ok", K


def uq_verify_attention(query, kc, ks, vc, vs, block_table, seq_lens, K, *, sm_scale=None, workspace=None, out=None,
                        rotate_q=False, tree_mask=None):
    """query [B*K, Hq, D] (uniform K per request, the varlen layout) -> [B*K, Hq, D] (reference uqmt/vllm_adapter.py:37-45).
    seq_lens counts all stored tokens including the K being verified.  workspace: fp32 scratch of
    uq_cuda.workspace_floats(...) elements (nothing is allocated inside then, out given).  rotate_q: the cache holds
    Hadamard-rotated keys (append_kv(rotate_k=True)), so the queries are rotated the same way first.  tree_mask
    int32 [B, K]: the draft tokens form a tree (uq_cuda.uq_tree_decode)."""
    BK, HQ, D = query.shape
    if K < 1 or BK % K:
        raise RuntimeError(f"{BK} query tokens are not a multiple of K={K}")
    B = BK // K
    q = query.reshape(B, K, HQ, D)
    if rotate_q:
        q = uq_cuda.fwht(q)
    o4 = None if out is None else out.view(B, K, HQ, D)
    nsplit = None
    if workspace is not None:   # the scratch bounds the number of partial slots: the usual count, or as many as the buffer holds
        nsplit = _slots_for(workspace, B, K, HQ, kc.shape[1], D, block_table.shape[1], query.device)
    if tree_mask is not None:
        o = uq_cuda.uq_tree_decode(q, kc, ks, vc, vs, block_table, seq_lens, tree_mask, sm_scale=sm_scale, out=o4, workspace=workspace, nsplit=nsplit)
    else:
        o = uq_cuda.uq_decode_cuda(q, kc, ks, vc, vs, block_table, seq_lens, sm_scale=sm_scale, out=o4, workspace=workspace, nsplit=nsplit)
    return o.reshape(BK, HQ, D)


def _slots_for(workspace, B, K, HQ, HKV, D, n_pages, device):
    want = uq_cuda.auto_nsplit(B, HKV, n_pages, torch.cuda.get_device_properties(device).multi_processor_count, K, HQ // HKV)
    while want > 1 and uq_cuda.workspace_floats(B, K, HQ, HKV, D, want) > workspace.numel():
        want -= 1
    if uq_cuda.workspace_floats(B, K, HQ, HKV, D, want) > workspace.numel():
        raise RuntimeError("scratch too small")
    return want


def append_kv(kc, ks, vc, vs, key, value, slot_mapping, *, rotate_k=False, rule="ceil", c=None, kernel=None):
    """Quantize new key/value [T, Hkv, D] and write them at flat slots (slot = physical_page * PAGE + offset), the
    cache-append hook of an engine (reference uqmt/vllm_adapter.py:48-59); one kernel launch, a decode step's tokens or a
    whole prompt's.  The keyword options are the reference's configurable quantiser (uqmt/quant.py): Hadamard-rotated keys and
    the 'paper' scale rule; `kernel` as in uq_cuda.append_kv."""
    uq_cuda.append_kv(kc, ks, vc, vs, key, value, slot_mapping, rotate_k=rotate_k, rule=rule, c=c, kernel=kernel)
