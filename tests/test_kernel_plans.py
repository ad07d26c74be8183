"""Launch geometry of the shared-box convolution kernels, swept on the CPU.

The planners are the host arithmetic the launchers themselves use (box sizes, stages, tap sets, pixel splits);
they need no device.  The sweep checks every invariant the kernels rely on: boxes and the rows their most shifted
views reach stay inside their shared-memory slots, stages fit the CTA's shared memory, accumulators fit tensor
memory, TMA boxes respect the 256-per-dimension limit, tiles and splits cover the problem exactly.
"""
import ctypes as C
import itertools

import pytest

from eagersgd_b200.parallel import _native as N

HALO_BYTES = 32 * 1024
STAGE_AREA = 161 * 1024


def _lib():
    lib = N.cuda()
    lib.esgd_conv2d_halo_plan.argtypes = [C.c_int] * 9 + [C.c_void_p]
    lib.esgd_conv2d_halo_plan.restype = None
    lib.esgd_conv2d_wgrad_halo_plan.argtypes = [C.c_int] * 9 + [C.c_void_p]
    lib.esgd_conv2d_wgrad_halo_plan.restype = None
    return lib


SHAPES = [(n, hw, cin, cout, k) for n, hw, cin, cout, k in itertools.product(
    (1, 7, 256), (7, 8, 14, 24, 28, 56, 112, 126, 130, 224), (64, 128, 256, 512), (64, 72, 128, 256, 512), (2, 3, 5, 7))]


def test_forward_halo_plans_fit_their_slots():
    lib = _lib()
    out = (C.c_int * 10)()
    seen = 0
    for n, hw, cin, cout, k in SHAPES:
        pad = (k - 1) // 2
        lib.esgd_conv2d_halo_plan(n, hw, hw, cin, cout, k, k, 1, pad, out)
        ok, bh, pw, bn, res_kb, nhalo, nst, box, view, used = list(out)
        if not ok:
            continue
        seen += 1
        ho, wo = hw + 2 * pad - k + 1, hw + 2 * pad - k + 1
        assert pw == wo + k - 1 and pw <= 128 and ho % bh == 0 and bh * pw <= 128
        assert bh * wo >= 64                                  # enough real rows per 128-row tile
        assert box <= HALO_BYTES and view <= HALO_BYTES       # the box and the farthest view stay in the slot
        assert pw <= 256 and bh + k - 1 <= 256                # TMA box extents
        assert used <= STAGE_AREA and nhalo in (2, 3) and nst >= 1
        assert bn in (64, 128) and cout <= 128
        if res_kb:
            assert res_kb == k * k * (cin // 64) and nhalo == 2
        else:
            assert nst >= 2
    assert seen > 50
    # stride 2 and wide outputs never take this path
    lib.esgd_conv2d_halo_plan(4, 56, 56, 64, 64, 3, 3, 2, 1, out)
    assert out[0] == 0
    lib.esgd_conv2d_halo_plan(4, 14, 14, 256, 256, 3, 3, 1, 1, out)
    assert out[0] == 0


@pytest.mark.parametrize("sms", [148, 132])
def test_weight_gradient_plans_cover_the_problem(sms):
    lib = _lib()
    out = (C.c_int * 16)()
    seen = 0
    for n, hw, cin, cout, k in SHAPES:
        pad = (k - 1) // 2
        lib.esgd_conv2d_wgrad_halo_plan(n, hw, hw, cin, cout, k, k, pad, sms, out)
        ok, bh, pw, ksteps, abox, xbox, nst, sets, tps, splits, bps, grid, bn, smem, mt, nt = list(out)
        if not ok:
            continue
        seen += 1
        ho = wo = hw + 2 * pad - k + 1
        assert ho % bh == 0 and bh * pw <= 128 and ksteps <= 8 and ksteps * 16 >= bh * pw
        assert abox % 1024 == 0 and xbox % 1024 == 0
        assert abox >= ksteps * 16 * 128 >= bh * pw * 128                       # dy box + zero K padding
        off_max = (k - 1) * pw + (k - 1)
        assert xbox >= (ksteps * 16 + off_max) * 128 >= (bh + k - 1) * pw * 128  # x box and the farthest view
        assert 2 <= nst <= 4 and nst * (2 * abox + (bn // 64) * xbox) + 1024 + 256 <= smem <= 227 * 1024
        assert tps * bn <= 512 and sets * tps >= k * k and (sets - 1) * tps < k * k   # accumulators fit TMEM, taps covered
        boxes = (ho // bh) * n
        assert splits * bps >= boxes and (splits - 1) * bps < boxes               # no empty split, all boxes covered
        assert grid == sets * mt * nt * splits and mt == -(-cout // 128) and nt == -(-cin // bn)
        assert pw <= 256 and bh + k - 1 <= 256
    assert seen > 100
