"""Two-GPU equivalence tests (NCCL): run only where at least two GPUs are visible.
Row sharding and the column split (with the all-gather, and with the epilogue writing into the peers' matrices)
must reproduce the single-GPU result bit for bit."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"      # plain peer stores only, no multicast objects
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import quarot_b200 as qb
        from quarot_b200 import dist as qd, synth
        M, K, N = 300, 4096, 2048
        x = synth.activations(M, K, seed=5).to(dev)
        w, sw = synth.weights(N, K, seed=6)
        w, sw = w.to(dev), sw.to(dev)
        quant = qb.nn.HadamardQuantizer(K)
        lin = qb.nn.Linear4bit(K, N).to(dev)
        lin.weight, lin.weight_scales = w, sw
        full = lin(quant(x))                                    # single-GPU result, computed on every rank
        # rows sharded, weights replicated, no collective on the data path
        a, b = qd.shard_rows(M, world, rank)
        local = lin(quant(x[a:b].contiguous()))
        rows_ok = torch.equal(qd.gather_rows(local, M), full)
        # output channels split, all-gather of the fp16 slabs
        col = qd.ColumnSplitLinear4bit(w, sw, None)
        cols_ok = torch.equal(col(quant(x)), full)
        # the same split with the epilogue storing straight into every rank's matrix (no all-gather)
        fused = qd.FusedColumnSplitLinear4bit(w, sw, None)
        target = qd.SymmetricOutput(M, N, dev)
        fused_ok = True
        for _ in range(3):
            got = fused(quant(x), target)
            torch.cuda.synchronize()
            fused_ok = fused_ok and bool(torch.equal(got, full))
        # few token rows: the fused module copies its slab into the peers' matrices instead
        xs = x[:24].contiguous()
        small = qd.SymmetricOutput(24, N, dev)
        fused_ok = fused_ok and bool(torch.equal(fused(quant(xs), small), lin(quant(xs))))
        ret[rank] = (bool(rows_ok), bool(cols_ok), bool(fused_ok))
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert dict(ret) == {0: (True, True, True), 1: (True, True, True)}
