"""Host mirrors of device tile schedules. The fused GEMM + reduce-scatter covers every tile exactly
once, keeps each tile inside its owner's row block and alternates owners along every CTA's tile
list; the persistent attention backward kernels visit every tile once, heaviest first, with
balanced totals per CTA."""
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


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("n_tiles", [0, 1, 2, 5, 8, 13])
def test_all_reduce_order_puts_own_tiles_last(world, n_tiles):
    from eth_b200.parallel.fused_tp import all_reduce_order
    for okey in range(2 * world):
        for rank in range(world):
            order = all_reduce_order(okey, n_tiles, world, rank)
            assert sorted(order) == list(range(n_tiles))          # a permutation of the list
            owners = [(okey + it) % world for it in order]
            dist = [(o - rank - 1) % world for o in owners]       # 0 for rank+1, ..., world-1 for own
            assert dist == sorted(dist)
            own = [it for it in order if (okey + it) % world == rank]
            assert own == sorted(own) and order[len(order) - len(own):] == own
        # a rank reaches its k-th own tile no earlier than any peer has pushed its partial of that
        # tile: position of the tile in the peer's order < number of peer-owned tiles of the owner
        for owner in range(world):
            own_pos = {it: pos for pos, it in enumerate(all_reduce_order(okey, n_tiles, world, owner))}
            for peer in range(world):
                if peer == owner:
                    continue
                peer_pos = {it: pos for pos, it in enumerate(all_reduce_order(okey, n_tiles, world, peer))}
                for it in range(n_tiles):
                    if (okey + it) % world == owner:
                        assert peer_pos[it] <= own_pos[it]


@pytest.mark.parametrize("ctas,tiles,pairs", [(148, 16, 64), (148, 8, 32), (148, 16, 3), (7, 5, 4), (148, 1, 10)])
def test_attention_backward_tile_order_covers_every_tile_once_and_is_balanced(ctas, tiles, pairs):
    from eth_b200.ops.functional import attention_backward_tile_order
    order = attention_backward_tile_order(ctas, tiles, pairs)
    seen = sorted((slot, pair) for lst in order for slot, pair, _ in lst)
    assert seen == [(s, p) for s in range(tiles) for p in range(pairs)]
    # every CTA walks its tiles heaviest first
    for lst in order:
        assert [w for _, _, w in lst] == sorted((w for _, _, w in lst), reverse=True)
    loads = [sum(w for _, _, w in lst) for lst in order]
    busy = [x for x in loads if x]
    # alternating the direction per round keeps the heaviest CTA within one heaviest tile of the mean
    assert max(busy) - sum(loads) / len(loads) <= tiles
    if (ctas, tiles, pairs) == (148, 16, 64):      # b4 h16 s2048: 67 vs 51 with plain round-robin
        assert max(loads) <= 61 and min(loads) >= 57
