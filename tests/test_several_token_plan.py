"""Host logic of the several-token decode kernel: how a weight is cut into k-slices and warp teams
(`wf_plan_several_tokens`, no device needed).  Every cut must cover K, fit shared memory and the partial-sum
buffer, use a team size the kernel knows, and keep every warp's work within a small factor of the even share."""
import ctypes
import itertools

import pytest

from warpforge_b200 import _native as N

QTYPES = {2: (128, 1152), 3: (128, 1280), 8: (128, 2176), 14: (256, 2368), 6: (128, 2176)}  # ggml type id: (tile k, tile bytes); Q5_0 runs as Q8_0
SHAPES = [(11008, 4096), (4096, 11008), (4096, 4096), (32000, 4096), (44032, 4096), (1024, 8192), (128, 8192), (3584, 8192),
          (1024, 28672), (16, 32), (7, 256), (100000, 256), (64, 131072)]


def _plan(qt, rows, k, cols, f32=0, sms=148):
    s, kc, team, part, smem = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int64()
    rc = N.load().wf_plan_several_tokens(qt, rows, k, cols, f32, sms, ctypes.byref(s), ctypes.byref(kc), ctypes.byref(team),
                                         ctypes.byref(part), ctypes.byref(smem))
    assert rc == N.WF_OK
    return s.value, kc.value, team.value, part.value, smem.value


@pytest.mark.parametrize("qt", sorted(QTYPES))
def test_every_cut_is_valid(qt):
    tk, tb = QTYPES[qt]
    for (rows, k), cols in itertools.product(SHAPES, (1, 3, 4, 8, 9, 16, 17, 30, 32)):
        if k % (256 if qt == 14 else 32):
            continue
        slices, kc, team, part, smem = _plan(qt, rows, k, cols)
        rt, kt = -(-rows // 16), -(-k // tk)
        if slices == 0:  # nothing fits: only allowed when even one slice per k-tile overflows the partial sums
            assert kt * cols * rt * 64 > (8 << 20) or cols * (tk * 2 + 64) > 200 * 1024, (qt, rows, k, cols)
            continue
        assert 1 <= slices <= min(kt, 64, 148) and kc >= 1
        assert (slices - 1) * kc < kt <= slices * kc, "the slices cover K exactly, the last one may be shorter"
        assert team in (1, 2, 3, 4, 5, 8, 16)
        assert smem <= 200 * 1024
        assert part == int(slices > 1)
        if part:
            assert slices * cols * rt * 64 <= (8 << 20)
        # the busiest warp: units of its team x its share of a unit's tiles, against the even share over 148 x 16 warps
        teams = 16 // team
        worst = 0
        for sl in range(slices):
            ctas = (148 - sl + slices - 1) // slices
            kcs = min(kc, kt - sl * kc)
            worst = max(worst, -(-(-(-rt // ctas)) // teams) * -(-kcs // team))
        even = rt * kt / (148 * 16)
        if kt <= 256:  # beyond 64 slices of K (K > 8192 k-tiles' worth per row-tile) the slice count is capped
            assert worst <= max(4.0 * even, even + 3), (qt, rows, k, cols, slices, kc, team, worst, even)


def test_fp32_tokens_always_use_partial_sums_and_bad_arguments_are_refused():
    slices, kc, team, part, _ = _plan(8, 4096, 4096, 3, f32=1)
    assert slices >= 1 and part == 1
    lib = N.load()
    z = ctypes.c_int()
    assert lib.wf_plan_several_tokens(2, 4096, 4096, 33, 0, 148, ctypes.byref(z), ctypes.byref(z), ctypes.byref(z), None, None) == N.WF_ERR_INVALID_ARGUMENT
    assert lib.wf_plan_several_tokens(12, 4096, 4096, 8, 0, 148, ctypes.byref(z), ctypes.byref(z), ctypes.byref(z), None, None) == N.WF_ERR_UNSUPPORTED_TYPE
    assert lib.wf_plan_several_tokens(2, 4096, 4096, 8, 0, 148, None, ctypes.byref(z), ctypes.byref(z), None, None) == N.WF_ERR_INVALID_ARGUMENT


def test_fewer_sms_still_cut_sensibly():
    for sms in (1, 8, 132):
        slices, kc, team, _, smem = _plan(2, 11008, 4096, 8, sms=sms)
        assert 1 <= slices <= sms and smem <= 200 * 1024
