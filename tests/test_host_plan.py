"""The strip schedule of the host-buffer entries (b200_sgemm_host_plan): pure host arithmetic, checked on CPU.

Row panels of A and column panels of B are uploaded alternately and every upload makes one rectangle of C
computable; the rectangles must tile C exactly once whatever the shape, start on multiples of the 128-wide CTA tile,
and only the small early rectangles may be split along K."""
import numpy as np
import pytest

SHAPES = [(4096, 4096, 4096), (1024, 1024, 1024), (1100, 1536, 1024), (2304, 1280, 1280), (16384, 2048, 16384),
          (5000, 1025, 3000), (1024, 9000, 1024), (130, 70, 33), (1, 1, 1), (1023, 4096, 4096), (4096, 4096, 1000)]


@pytest.mark.parametrize("pipelined", [False, True], ids=["single", "pipelined"])
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_strips_tile_c_exactly_once(sgemm, shape, pipelined):
    M, N, K = shape
    plan = sgemm.host_plan(M, N, K, 148, pipelined)
    cover = np.zeros((-(-M // 64), -(-N // 64)), dtype=np.int32)  # 64-granular is enough: strips start on multiples of 128
    for (r0, rn, c0, cn), split in plan:
        assert rn > 0 and cn > 0 and r0 + rn <= M and c0 + cn <= N
        assert r0 % 128 == 0 and c0 % 128 == 0
        assert 1 <= split <= 16 and (split == 1 or K // split >= 512)
        cover[r0 // 64:-(-(r0 + rn) // 64), c0 // 64:-(-(c0 + cn) // 64)] += 1
    assert (cover == 1).all()
    big = M >= 1024 and N >= 1024 and K >= 1024
    if not big:
        assert len(plan) == 1
    elif not pipelined:
        assert 1 < len(plan) <= 15
    else:
        assert 1 <= len(plan) <= 15 and len(plan) <= len(sgemm.host_plan(M, N, K, 148))


def test_4096_cube_pipelined_schedule(sgemm):
    """A job submitted while another is in flight: two pieces per operand, three strips of 256, 256 and 512 tiles."""
    plan = sgemm.host_plan(4096, 4096, 4096, 148, pipelined=True)
    assert plan == [((0, 2048, 0, 2048), 1), ((2048, 2048, 0, 2048), 1), ((0, 4096, 2048, 2048), 1)]


def test_4096_cube_schedule(sgemm):
    plan = sgemm.host_plan(4096, 4096, 4096, 148)
    assert len(plan) == 15  # 8 + 8 uploads, the first one computes nothing
    assert plan[0] == ((0, 512, 0, 512), 8)          # 16 tiles: split so that every SM has work
    assert plan[1] == ((512, 512, 0, 512), 8)
    assert plan[2] == ((0, 1024, 512, 512), 4)
    assert plan[-1] == ((0, 4096, 3584, 512), 1)     # the last column panel against all of A
    assert sum(rn * cn for (r0, rn, c0, cn), _ in plan) == 4096 * 4096
    # splits only while a strip has fewer tiles than half the SMs
    for (r0, rn, c0, cn), split in plan:
        tiles = -(-rn // 128) * -(-cn // 128)
        assert (split > 1) == (2 * tiles <= 148)


def test_plan_argument_errors(sgemm):
    with pytest.raises(sgemm.SgemmError):
        sgemm.host_plan(0, 4, 4)
    with pytest.raises(sgemm.SgemmError):
        sgemm.host_plan(4, 4, 4, 0)
