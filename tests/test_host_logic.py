"""Host-side logic that needs no GPU: dependency flags of a decode program, workload byte counts."""
from warpforge_b200 import quant as Q
from warpforge_b200.decode import LLAMA_70B_Q4_K, LLAMA_7B_Q4_0, ProjectionStack, StackSpec


def _stack(spec, layers):
    st = ProjectionStack.__new__(ProjectionStack)  # no context, no device memory: only the bookkeeping
    st.spec, st.layers = spec, layers
    return st


def test_program_flags_follow_the_layer_structure():
    new = ProjectionStack.OP_NEW_X | ProjectionStack.OP_DEPENDS
    # Wq Wk Wv share one input; Wo, Wgate (+Wup), Wdown each read what the previous group produced
    assert _stack(LLAMA_7B_Q4_0, 2).op_flags() == [new, 0, 0, new, new, 0, new] * 2
    assert _stack(LLAMA_70B_Q4_K, 1).op_flags() == [new, 0, 0, new, new, 0, new]


def test_program_flags_follow_the_input_buffer():
    # unknown names: a projection whose k differs from its predecessor's reads another buffer and must stage anew
    spec = StackSpec("t", Q.QuantizationType.Q4_0, 1, (("a", 512, 256), ("b", 256, 256), ("c", 256, 512)), 0)
    new = ProjectionStack.OP_NEW_X | ProjectionStack.OP_DEPENDS
    assert _stack(spec, 1).op_flags() == [new, 0, new]


def test_bytes_per_token_of_the_7b_stack():
    # 32 layers x (4 x [4096x4096] + 2 x [11008x4096] + [4096x11008]) Q4_0 blocks of 18 bytes per 32 weights
    per_layer = (4 * 4096 * 4096 + 3 * 11008 * 4096) // 32 * 18
    assert LLAMA_7B_Q4_0.bytes_per_token() == 32 * per_layer == 3642753024


def test_benchmark_entry_points_import_without_a_gpu():
    """bench.py and the helper benchmarks only touch the device inside main(): importing them (what the driver's
    build check and `--help` do) must work on a machine without a GPU."""
    import importlib

    for name in ("bench", "warpforge_b200.bench_config5", "warpforge_b200.bench_glue"):
        mod = importlib.import_module(name)
        assert callable(mod.main)


def test_config5_shard_arithmetic():
    """One rank's shard of the 70B-shape layer: 60 162 048 bytes of Q4_K blocks (4 812 963 840 per GPU over 80 layers,
    the figure of benchmark config 5) and 106 954 752 weights."""
    from warpforge_b200.decode import LLAMA_70B_Q4_K as spec

    per_layer = sum((rows // 8) * spec.qtype.row_bytes(k) for _, rows, k in spec.projections)
    assert per_layer == 60162048 and per_layer * spec.layers == 4812963840
    assert sum((rows // 8) * k for _, rows, k in spec.projections) == 106954752
