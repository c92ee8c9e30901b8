"""Host logic of the two multi-GPU modes, run as world_size-2 gloo ranks on CPU (no GPU needed): the shard arithmetic,
the all-gather and the merge order are the library's; the per-shard attention is the CPU oracle standing in for the
CUDA entry points."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from tests.cases import load_cases


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_partial(q, kc, ks, vc, vs, bt, sl, off, nsplit=None, sm_scale=None):
    from oracle import uq_oracle as O
    PAGE = kc.shape[2]
    nloc = np.clip(sl.numpy() - off.numpy(), 0, bt.shape[1] * PAGE).astype(np.int32)
    o, lse = O.reference(q.view(torch.int16).numpy().view(np.uint16), kc.numpy(), ks.numpy(), vc.numpy(), vs.numpy(), bt.numpy(), sl.numpy(),
                         sm_scale, pos_offset=off.numpy(), n_local=nloc, return_lse=True)
    return torch.from_numpy(o), torch.from_numpy(lse / np.log(2.0)).float()   # the CUDA partial reports log2


def _oracle_merge(o_all, l_all):
    from oracle import uq_oracle as O
    return torch.from_numpy(O.merge(o_all.numpy(), l_all.numpy() * np.log(2.0)))


def _rank(rank, world, port, name, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from all_quant_b200 import uq_cuda
        from oracle import uq_oracle as O
        c = [x for x in load_cases() if x.name == name][0]
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
        q = t(c.q.view(np.int16)).view(torch.bfloat16)
        kc, ks, vc, vs, bt, sl = (t(a) for a in (c.kc, c.ks, c.vc, c.vs, c.bt, c.sl))
        # mode (b): context split
        bt_loc, off = uq_cuda.context_shard(bt, rank, world, c.PAGE)
        got = uq_cuda.uq_decode_context_split(q, kc, ks, vc, vs, bt_loc, sl, off, partial_fn=_oracle_partial, merge_fn=_oracle_merge,
                                              sm_scale=c.sm_scale)
        err_b = float(np.abs(got.numpy() - c.ref).max())
        # mode (a): head partition, no collective on the data path; the gather below is only this test's check
        qh, kch, ksh, vch, vsh = uq_cuda.head_shard(q, kc, ks, vc, vs, rank, world)
        mine = torch.from_numpy(O.reference(qh.view(torch.int16).numpy().view(np.uint16), kch.numpy(), ksh.numpy(), vch.numpy(), vsh.numpy(),
                                            bt.numpy(), sl.numpy(), c.sm_scale))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        err_a = float(np.abs(torch.cat(parts, dim=2).numpy() - c.ref).max())
        if rank == 0:
            out.put((err_a, err_b))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["gen_d256_K8", "gen_k8g8_K8"])
def test_two_ranks_head_partition_and_context_split(name):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, name, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    err_a, err_b = out.get(timeout=10)
    assert err_a <= 2e-5 and err_b <= 2e-5, (err_a, err_b)


def test_shard_arithmetic():
    from all_quant_b200 import uq_cuda
    bt = torch.arange(2 * 7, dtype=torch.int32).reshape(2, 7)
    seen = []
    for r in range(4):
        b, off = uq_cuda.context_shard(bt, r, 4, 64)
        assert b.shape == (2, 2) and off.tolist() == [min(r * 2, 7) * 64] * 2
        seen.append(b[:, : max(0, min(7, (r + 1) * 2) - r * 2)])
    assert torch.equal(torch.cat(seen, 1), bt)
    with pytest.raises(ValueError):
        uq_cuda.head_shard(torch.zeros(1, 1, 6, 32), *(torch.zeros(1, 3, 16, 16),) * 4, 0, 2)
