"""The one-token program with the fp32 operations between a decoder layer's projections fused into it
(rms_norm into the staging of Wq/Wk/Wv and Wgate/Wup, silu * up into the staging of Wdown, the residual adds into
the stores of Wo and Wdown) against the CPU oracle running the same layer op by op: rms_norm
(cpu/ops/scalar/CustomCallKernel.java:173-224), the quantized linear, silu and multiply (:262-280), add.
Every intermediate buffer of every layer is compared, so an error cannot hide behind a later normalisation."""
import numpy as np
import pytest

from oracle import oracle as O
from warpforge_b200 import quant as Q

pytestmark = pytest.mark.gpu

OQ = {"Q4_0": O.Q4_0, "Q4_K": O.Q4_K, "Q8_0": O.Q8_0}


def _oracle_layers(orc, st):
    """name -> expected fp32 row, for every buffer the program writes."""
    want, h = {}, st.host["h0"]
    oq, nt = OQ[st.qtype.name], orc.max_threads()

    def lin(l, name, x):
        rows, k = st.shapes[name]
        return orc.qlinear(oq, st.blocks[l][name], rows, k, x.reshape(1, k), nthreads=nt).reshape(rows)

    for l in range(st.layers):
        x1 = orc.rms_norm(h.reshape(1, -1), st.host[f"gamma1_{l}"], st.eps).reshape(-1)
        for n, w in (("q", "wq"), ("k", "wk"), ("v", "wv")):
            want[f"{n}_{l}"] = lin(l, w, x1)
        hmid = orc.add(h, lin(l, "wo", st.host[f"attn_{l}"]))
        want[f"hmid_{l}"] = hmid
        x2 = orc.rms_norm(hmid.reshape(1, -1), st.host[f"gamma2_{l}"], st.eps).reshape(-1)
        gate, up = lin(l, "wgate", x2), lin(l, "wup", x2)
        want[f"gate_{l}"], want[f"up_{l}"] = gate, up
        h = orc.add(hmid, lin(l, "wdown", orc.swiglu(gate, up)))
        want[f"h{l + 1}"] = h
    return want


@pytest.mark.parametrize("qt,d,ffn,layers", [(Q.QuantizationType.Q4_0, 512, 1408, 3), (Q.QuantizationType.Q4_K, 1024, 2816, 2),
                                             (Q.QuantizationType.Q8_0, 256, 640, 2)])
def test_fused_layers_match_the_oracle_op_by_op(oracle, qt, d, ffn, layers):
    from warpforge_b200.backend import CudaContext
    from warpforge_b200.decode import FusedDecoderStack

    if qt == Q.QuantizationType.Q4_K:
        ffn = (ffn // 256) * 256
    ctx = CudaContext(0)
    try:
        st = FusedDecoderStack(ctx, qt, d, ffn, layers, seed=5)
        st.run()
        ctx.synchronize()
        first = {n: st.read(n) for n in st.dev if n.split("_")[0] in ("q", "k", "v", "hmid", "gate", "up") or (n[0] == "h" and n[1:].isdigit() and n != "h0")}
        want = _oracle_layers(oracle, st)
        assert set(want) == set(first)
        for name, w in want.items():
            got = first[name]
            assert np.isfinite(got).all(), name
            rel = float(np.max(np.abs(got - w)) / np.max(np.abs(w)))
            assert rel <= 1e-3, f"{name}: max err / max|y| = {rel:.3e}"
        st.run()  # the same token again: the residual stream starts from h0 again, so the same bits must come out
        ctx.synchronize()
        for name, a in first.items():
            assert np.array_equal(st.read(name).view(np.uint32), a.view(np.uint32)), name + ": not the same bits from run to run"
        st.close()
    finally:
        ctx.close()


def test_fused_kinds_are_refused_for_several_tokens():
    from warpforge_b200 import _native as N
    from warpforge_b200.backend import CudaContext, QuantizedWeight
    import ctypes

    ctx = CudaContext(0)
    try:
        w = QuantizedWeight(ctx, Q.QuantizationType.Q4_0, Q.synth_q4_0(64, 256, 1), 64, 256)
        x, y = ctx.allocate(4 * 256 * 4), ctx.allocate(4 * 64 * 4)
        arr = lambda v, t: (t * len(v))(*v)
        prog = ctypes.c_int64()
        rc = ctx._lib.wf_program_create_fused(ctx.handle, 1, arr([w.handle], ctypes.c_int64), arr([x], ctypes.c_int64), arr([y], ctypes.c_int64),
                                              arr([1], ctypes.c_int), arr([N.WF_X_F32], ctypes.c_int), None, None, None, 4, 1, 0, None, ctypes.byref(prog))
        assert rc == N.WF_ERR_SHAPE and prog.value == 0
        w.close()
    finally:
        ctx.close()
