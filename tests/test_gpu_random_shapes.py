"""Seeded random shapes through the operator: row counts around the 16-row tile and far from it, K from one block
to 16384, 1 - 40 bf16 tokens or 1 - 11 fp32 tokens, every block type -- whichever kernel the call lands on
(one token, several tokens in one or more launches, tensor-core GEMM above 32) must agree with the CPU oracle to
1e-3 of the output's largest magnitude."""
import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

TYPES = [(Q.QuantizationType.Q4_0, O.Q4_0), (Q.QuantizationType.Q8_0, O.Q8_0), (Q.QuantizationType.Q4_K, O.Q4_K),
         (Q.QuantizationType.Q4_1, O.Q4_1), (Q.QuantizationType.Q5_0, O.Q5_0)]


@pytest.mark.parametrize("seed", [1, 2, 3, 4])
def test_random_shapes_match_the_oracle(oracle, seed):
    from warpforge_b200.backend import DotGeneralOp, LINEAR_DIMS, NvidiaBackend, Tensor

    be = NvidiaBackend(0)
    rng = np.random.default_rng(seed)
    try:
        for it in range(40):
            qt, oq = TYPES[rng.integers(len(TYPES))]
            blk = 256 if qt == Q.QuantizationType.Q4_K else 32
            rows = int(rng.choice([1, 7, 16, 17, 100, 128, 129, 500, 1000, 3000, 5000]))
            k = blk * int(rng.integers(1, 16384 // blk // (4 if rows > 1000 else 1) + 1))
            f32 = rng.random() < 0.25
            m = int(rng.integers(1, 12 if f32 else 41))
            blocks = Q.synth_weight(qt, rows, k, 1000 * seed + it)
            w = be.upload_weight(qt, blocks, rows, k)
            if f32:
                xf = Q.synth_activation_f32(m, k, 2000 * seed + it)
                xt = Tensor.from_float_array(xf)
            else:
                xb = Q.synth_activation_bf16(m, k, 2000 * seed + it)
                xt, xf = Tensor.from_bf16_bits(xb), Q.bf16_bits_to_float(xb)
            got = be.execute(DotGeneralOp(LINEAR_DIMS, (m, rows)), [xt, w])[0].data
            want = oracle.qlinear(oq, blocks, rows, k, xf, nthreads=oracle.max_threads())
            rel = float(np.max(np.abs(got - want)) / max(float(np.max(np.abs(want))), 1e-30))
            assert np.isfinite(got).all() and rel <= 1e-3, f"{qt.name} [{rows} x {k}], {m} {'fp32' if f32 else 'bf16'} tokens: {rel:.3e}"
            w.close()
    finally:
        be.close()
