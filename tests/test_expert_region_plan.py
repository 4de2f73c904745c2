"""The expert GEMM task keeps the operands of the step it computes and of the step it prefetches in two regions of
the activation tile, placed by a few lines of arithmetic in `run_moe_gemm` (mirage_b200/csrc/megakernel.cu): the next
region goes behind the current one if it fits, else to the front if it fits in front of the current one, else the step
is staged only after the current one is done.  This restates that arithmetic and checks, for random token counts per
expert and for the tile sizes the graph compiler hands out, that the two live regions never overlap and never leave
the tile -- the property the asynchronous copies rely on."""
import random

import pytest

ROW_PAD = 16


def align16(v):
    return (v + 15) & ~15


def region_bytes(cnt, xstride, ng, rows):
    n = max(cnt, 1)
    return align16(n * xstride) + 4 * ((n * ng + 3) & ~3) + align16(4 * rows * ng)


def host_tile_bytes(ntok, kt, fp8, task_rows=64):
    """moe_fp8_tile_bytes / the bf16 form of task_graph.cpp (the buffer the compiler reserves for `ntok` tokens)."""
    if not fp8:
        return ntok * (kt * 2 + ROW_PAD)
    return ntok * (kt + ROW_PAD) + 16 + 4 * (ntok * (kt // 128) + 4) + 4 * task_rows * (kt // 128) + 16


@pytest.mark.parametrize("ntok,kt,fp8,rows", [(16, 3584, True, 28), (32, 3584, True, 28), (64, 1024, True, 64), (8, 2048, True, 49),
                                               (16, 768, False, 16), (64, 1024, False, 32), (1, 7168, True, 28)])
def test_regions_stay_inside_the_tile_and_apart(ntok, kt, fp8, rows):
    esz = 1 if fp8 else 2
    xstride = kt * esz + ROW_PAD
    ng = kt // 128 if fp8 else 0
    tile = (host_tile_bytes(ntok, kt, fp8) + 255) // 256 * 256          # x_tile_bytes is rounded up to 256
    rng = random.Random(ntok * 1000 + kt)
    for trial in range(200):
        counts = [rng.choice([0, 1, 1, 2, 3, ntok // 2, ntok]) for _ in range(rng.randint(1, 40))]
        counts = [min(c, ntok) for c in counts]
        off, cnt = 0, counts[0]
        assert region_bytes(cnt, xstride, ng, rows) <= tile             # the first step is staged at offset 0
        for nxt in counts[1:]:
            need_c, need_n = region_bytes(cnt, xstride, ng, rows), region_bytes(nxt, xstride, ng, rows)
            off_n, ahead = off + need_c, True
            if off_n + need_n > tile:
                off_n = 0
                if need_n > off:
                    ahead = False
            assert off_n + need_n <= tile
            if ahead:                                                   # copied while the current region is being read
                assert off_n >= off + need_c or off_n + need_n <= off
            off, cnt = off_n, nxt
