"""GPU parity on benchmark config 5 (70B-shape projection set, Q4_K, row-sharded over 8 ranks): one
rank's shard of every projection shape, as a batch-16 decode step and as a 2048-token prefill,
through the C ABI against the CPU oracle.  Both run on the tensor-core GEMM (more than 8 bf16
tokens), so the bars are the GEMM's: max|d| / max|y| <= 1e-3 and rms(d) / rms(y) <= 3e-4.  The
oracle checks sampled weight rows at these sizes; repeat calls must give the same bits."""
import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

WORLD = 8
# (name, rows of the unsharded weight, k): d_model 8192, 64 query / 8 KV heads of 128, FFN 28672
SHAPES = [("wq", 8192, 8192), ("wk", 1024, 8192), ("wo", 8192, 8192), ("wgate", 28672, 8192), ("wdown", 8192, 28672)]


@pytest.fixture(scope="module")
def backend():
    from warpforge_b200.backend import NvidiaBackend

    b = NvidiaBackend(0)
    yield b
    b.close()


def _gemm(backend, w, xb):
    from warpforge_b200.backend import DotGeneralOp, LINEAR_DIMS, Tensor

    return backend.execute(DotGeneralOp(LINEAR_DIMS, (xb.shape[0], w.rows)), [Tensor.from_bf16_bits(xb), w])[0].data


def _check(got, want):
    d = got.astype(np.float64) - want.astype(np.float64)
    rel_max = float(np.max(np.abs(d)) / np.max(np.abs(want)))
    rel_rms = float(np.sqrt(np.mean(d * d)) / np.sqrt(np.mean(want.astype(np.float64) ** 2)))
    assert rel_max <= 1e-3 and rel_rms <= 3e-4, f"max err / max|y| = {rel_max:.3e}, rms err / rms y = {rel_rms:.3e}"


@pytest.mark.parametrize("name,rows,k", SHAPES)
@pytest.mark.parametrize("tokens,sampled", [(16, 256), (2048, 16)])
def test_config5_rank_shard(backend, oracle, name, rows, k, tokens, sampled):
    shard = rows // WORLD  # rank 3's rows, uploaded as a weight of its own (what every rank does)
    seed = Q.config_seed(5, rows + k)
    blocks = Q.synth_q4_k(shard, k, seed)
    xb = Q.synth_activation_bf16(tokens, k, seed + tokens)
    w = backend.upload_weight(Q.QuantizationType.Q4_K, blocks, shard, k)
    got = _gemm(backend, w, xb)
    assert got.shape == (tokens, shard)
    rng = np.random.default_rng(seed)
    pick = np.sort(rng.choice(shard, min(sampled, shard), replace=False))
    want = oracle.qlinear_rows(O.Q4_K, blocks, k, Q.bf16_bits_to_float(xb), pick, nthreads=oracle.max_threads())
    _check(got[:, pick], want)
    again = _gemm(backend, w, xb)
    assert np.array_equal(got.view(np.uint32), again.view(np.uint32))
    w.close()
