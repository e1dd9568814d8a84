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
