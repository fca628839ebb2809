"""Multi-rank host logic on CPU ranks (gloo, world size 2): row sharding and the column split
with its all-gather.  The local compute is the oracle, injected; no GPU is involved."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import quarot_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_linear(q, sx, w, sw, bias):
    acc = O.matmul_i4(q.reshape(-1, q.shape[-1]), w)
    out = O.sym_dequant_fp32(acc, sx.reshape(-1), sw).half()
    if bias is not None:
        out = out + bias
    return out.reshape(*q.shape[:-1], w.shape[0])


def _worker(rank, world, port, mode, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import quarot_b200 as qb
        from quarot_b200 import dist as qd, synth
        M, K, N = 37, 256, 64
        x = synth.activations(M, K, seed=5)
        w, sw = synth.weights(N, K, seed=6)
        bias = (torch.arange(N) % 7 - 3).half() * 0.25
        s = O.quantizer_scales(x)
        q = O.pack_i4(O.sym_quant_codes(x, s))
        full = _oracle_linear(q, s, w, sw, bias)
        if mode == "rows":
            a, b = qd.shard_rows(M, world, rank)
            local = _oracle_linear(q[a:b], s[a:b], w, sw, bias)
            got = qd.gather_rows(local, M)
            ret[rank] = bool(torch.equal(got, full)) and (b - a) in (18, 19)
        elif mode == "columns":
            lin = qd.ColumnSplitLinear4bit(w, sw, bias, compute=_oracle_linear)
            assert lin.weight.shape == (N // world, K // 2) and lin.bias.shape == (N // world,)
            got = lin(qb.PackedQuantizedTensor(q.view(1, M, K // 2), s.view(1, 1, M)))
            ret[rank] = bool(torch.equal(got.view(M, N), full)) and got.shape == (1, M, N)
        elif mode == "bad_rows":
            try:
                qd.gather_rows(torch.zeros(3, 4), M)
                ret[rank] = False
            except RuntimeError:
                ret[rank] = True
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["rows", "columns", "bad_rows"])
def test_two_rank_gloo(mode):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, ret), nprocs=world, join=True)
    assert dict(ret) == {0: True, 1: True}


def test_shard_rows_partition():
    from quarot_b200 import dist as qd
    for m in (1, 7, 2048, 4099):
        for g in (1, 2, 4, 8):
            spans = [qd.shard_rows(m, g, r) for r in range(g)]
            assert spans[0][0] == 0 and spans[-1][1] == m
            assert all(spans[i][1] == spans[i + 1][0] for i in range(g - 1))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        qd.shard_rows(4, 2, 2)
    with pytest.raises(ValueError):
        qd.split_columns(torch.zeros(6, 4), torch.zeros(6, 1), None, 4, 0)
