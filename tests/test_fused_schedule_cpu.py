"""The tile schedule of the fused GEMM + reduce-scatter covers every tile exactly once, keeps each
tile inside its owner's row block and alternates owners along every CTA's tile list."""
import pytest

from eth_b200.parallel.fused_tp import reduce_scatter_schedule


@pytest.mark.parametrize("world,grid,tiles_m,tiles_n", [(2, 148, 64, 8), (4, 148, 64, 16), (8, 144, 64, 8), (2, 16, 4, 3),
                                                        (2, 148, 2, 1)])
def test_reduce_scatter_schedule_is_a_partition(world, grid, tiles_m, tiles_n):
    seen = {}
    for cta in range(grid):
        it, owners = 0, []
        while True:
            t = reduce_scatter_schedule(cta, grid, it, tiles_m, tiles_n, world)
            if t is None:
                break
            owner, tm, tn = t
            assert owner == (cta + it) % world
            assert owner * (tiles_m // world) <= tm < (owner + 1) * (tiles_m // world)
            assert (tm, tn) not in seen, f"tile {(tm, tn)} visited twice"
            seen[(tm, tn)] = (cta, it)
            owners.append(owner)
            it += 1
        assert all(a != b for a, b in zip(owners, owners[1:])) or world == 1
    assert len(seen) == tiles_m * tiles_n
