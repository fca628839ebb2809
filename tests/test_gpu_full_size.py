"""The benchmark configurations at their full sizes, CUDA path against the CPU oracle.

Prefill (LLaMA-2-7B at M = 2048, LLaMA-2-70B at M = 4096, every linear of a decoder layer): the oracle cannot
recompute 10^9 accumulators in seconds, so each shape is checked through
  * a checksum identity over ALL accumulators: sum_mn C[m,n] == sum_k (sum_m A[m,k]) (sum_n B[n,k]), exact in int64;
  * every 37th / 97th token row in full against the oracle: Hadamard output within 1e-3 of the fp32 operator, scales
    and int4 codes bit-exact given the kernel's own fp16 Hadamard output, int32 accumulators bit-exact, fused fp16
    output bit-equal to fp16(float(acc) * (s_x * s_w)) -- which is within 1e-2 of the fp32 reference by construction.
Decode (the four 7B shapes at M = 1, 8, 32, 64): every output against the oracle.
"""
import pytest
import torch

import quarot_b200 as qb
from quarot_b200 import _lib, synth
from quarot_b200.functional import hadamard as FH
from oracle import quarot_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _colsum_unpacked(packed, chunk=4096):
    """Column sums of the unpacked int4 matrix, int64 [K], computed on the CPU in row chunks."""
    total = torch.zeros(packed.shape[1] * 2, dtype=torch.int64)
    for r in range(0, packed.shape[0], chunk):
        total += O.unpack_i4(packed[r:r + chunk]).sum(0, dtype=torch.int64)
    return total


def _oracle_rows_matmul(a_rows, w, chunk=8192):
    """int32 accumulators of a few token rows against all N weight rows, N processed in chunks (bounded memory)."""
    return torch.cat([O.matmul_i4(a_rows, w[r:r + chunk]) for r in range(0, w.shape[0], chunk)], dim=1)


def _check_prefill_linear(M, K, N, had, seed, every):
    x = synth.activations_device(M, K, seed=seed, device=DEV)
    w_dev, sw_dev = synth.weights_device(N, K, seed=seed + 1, device=DEV)
    w, sw = w_dev.cpu(), sw_dev.cpu()
    khad = FH.get_hadK(K)[1] if had else 0
    table = FH.device_table(khad, DEV) if khad > 1 else None
    q, s, y = qb.hadamard_quant(x, table, khad, 1.0, return_y=True)
    acc = qb.matmul(q, w_dev)
    out = qb.linear_i4(q, s, w_dev, sw_dev)
    torch.cuda.synchronize()
    rows = torch.arange(0, M, every)
    qc, sc = q.cpu(), s.cpu()
    # kernel (a) on the sampled rows
    if had:
        y_ref = O.hadamard(x.cpu()[rows].float())
        err = (y.cpu()[rows].float() - y_ref).abs().amax(dim=1) / y_ref.abs().amax(dim=1)
        assert float(err.max()) < 1e-3                      # tolerance of the Hadamard output
        y_rows = y.cpu()[rows]
    else:
        y_rows = x.cpu()[rows]
    s_ref = O.quantizer_scales(y_rows)
    assert torch.equal(sc[rows], s_ref)
    assert torch.equal(qc[rows], O.pack_i4(O.sym_quant_codes(y_rows, s_ref)))
    # kernel (b): checksum over every accumulator, then the sampled rows in full
    want_sum = int((_colsum_unpacked(qc) * _colsum_unpacked(w)).sum())
    assert int(acc.sum(dtype=torch.int64)) == want_sum
    acc_ref = _oracle_rows_matmul(qc[rows], w)
    assert torch.equal(acc.cpu()[rows], acc_ref)
    assert torch.equal(out.cpu()[rows], O.sym_dequant_fp32(acc_ref, s_ref, sw).half())
    # the fused epilogue and the int32 path describe the same matrix everywhere, not only on the sampled rows
    deq = (acc.float() * (s.float().view(-1, 1) * sw_dev.float().view(1, -1))).half()
    assert torch.equal(out, deq)
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("name,K,N,had", synth.LLAMA2_7B)
def test_llama2_7b_prefill_linear_full_size(name, K, N, had):
    _check_prefill_linear(2048, K, N, had, seed=100 + K % 97 + N % 89, every=37)


@pytest.mark.parametrize("name,K,N,had", synth.LLAMA2_70B)
def test_llama2_70b_prefill_linear_full_size(name, K, N, had):
    _check_prefill_linear(4096, K, N, had, seed=200 + K % 97 + N % 89, every=97)


@pytest.mark.parametrize("M", [1, 8, 32, 64])
@pytest.mark.parametrize("name,K,N,had", synth.LLAMA2_7B)
def test_llama2_7b_decode_linear_against_oracle(name, K, N, had, M):
    """Decode-sized M: whichever kernel serves the shape (weight streaming, tensor cores with or without the
    split K loop, quantiser inside the kernel), every output value equals the oracle's."""
    x = synth.activations(M, K, seed=300 + M + N % 89)
    w, sw = synth.weights(N, K, seed=301 + N % 89)
    khad = FH.get_hadK(K)[1] if had else 0
    table = FH.device_table(khad, DEV) if khad > 1 else None
    xd, wd, swd = x.to(DEV), w.to(DEV), sw.to(DEV)
    q, s, y = qb.hadamard_quant(xd, table, khad, 1.0, return_y=True)
    y_cpu = y.cpu() if had else x
    if had:
        y_ref = O.hadamard(x.float())
        assert float(((y_cpu.float() - y_ref).abs().amax(dim=1) / y_ref.abs().amax(dim=1)).max()) < 1e-3
    s_ref = O.quantizer_scales(y_cpu)
    q_ref = O.pack_i4(O.sym_quant_codes(y_cpu, s_ref))
    assert torch.equal(s.cpu(), s_ref) and torch.equal(q.cpu(), q_ref)
    acc_ref = O.matmul_i4(q_ref, w)
    want = O.sym_dequant_fp32(acc_ref, s_ref, sw).half()
    assert torch.equal(qb.matmul(q, wd).cpu(), acc_ref)
    assert torch.equal(qb.linear_i4(q, s, wd, swd).cpu(), want)                          # cached workspace
    assert torch.equal(qb.linear_i4(q, s, wd, swd, use_workspace=False).cpu(), want)     # single pass
    if not had:
        # Sequential(Quantizer, Linear4bit) as one module: for the smallest M the quantiser runs inside the GEMV
        lin = qb.nn.Linear4bit(K, N).to(DEV)
        lin.weight, lin.weight_scales = wd, swd
        fused = qb.nn.fused.QuantLinear4bit(qb.nn.Quantizer(), lin)
        assert torch.equal(fused(xd).cpu(), want)
    assert _lib.kernel_status() == 0
