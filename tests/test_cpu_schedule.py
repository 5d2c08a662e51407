"""Schedule properties, enumerated on the CPU from the same header the kernels use."""
import itertools

import pytest

from penny_b200.parallel import schedule


@pytest.mark.parametrize("world", [2, 3, 4, 6, 8])
def test_stride_rings_are_hamiltonian(world):
    seen = set()
    for route in range(8):
        order = schedule.ring_order(world, 1, route)
        assert sorted(order) == list(range(world))
        seen.add(tuple(order))
    if world == 8:
        assert len(seen) == 4  # strides 1, 7, 3, 5


@pytest.mark.parametrize("world,nnodes", [(8, 2), (8, 4), (4, 2), (6, 2), (6, 3)])
def test_node_aware_rings(world, nnodes):
    gpn = world // nnodes
    for route in range(2 * max(1, gpn // 2)):
        order = schedule.ring_order(world, nnodes, route)
        assert sorted(order) == list(range(world))
        # a ring crosses each node boundary exactly once per lap
        crossings = sum(1 for i in range(world) if order[i] // gpn != order[(i + 1) % world] // gpn)
        assert crossings == nnodes
    # odd routes are the even ring walked backwards
    fwd, bwd = schedule.ring_order(world, nnodes, 0), schedule.ring_order(world, nnodes, 1)
    assert bwd == [fwd[(world - p) % world] for p in range(world)]
    if gpn >= 4:
        # different ring pairs leave a node from different local ranks
        exit0 = [fwd[i] % gpn for i in range(world) if fwd[i] // gpn != fwd[(i + 1) % world] // gpn]
        o2 = schedule.ring_order(world, nnodes, 2)
        exit2 = [o2[i] % gpn for i in range(world) if o2[i] // gpn != o2[(i + 1) % world] // gpn]
        assert set(exit0).isdisjoint(exit2)


@pytest.mark.parametrize("n", [2, 3, 4, 6, 8])
def test_ring_steps_pair_up_and_cover(n):
    """What position p sends at step s is what p+1 receives at step s, every chunk
    is reduced exactly n-1 times and every rank ends with every chunk."""
    have = [{c: {p} for c in range(n)} for p in range(n)]  # contributions folded into chunk c at position p
    complete = [set() for _ in range(n)]
    for step in range(2 * (n - 1)):
        sends = {}
        for p in range(n):
            sc, rc, reduce = schedule.ring_step_chunks(n, p, step)
            sends[p] = (sc, reduce)
        for p in range(n):
            sc, rc, reduce = schedule.ring_step_chunks(n, p, step)
            prev = (p - 1) % n
            assert sends[prev][0] == rc, "receive schedule must match the predecessor's send schedule"
        new = [dict(h) for h in have]
        for p in range(n):
            _, rc, reduce = schedule.ring_step_chunks(n, p, step)
            prev = (p - 1) % n
            incoming = have[prev][rc]
            if reduce:
                assert have[p][rc].isdisjoint(incoming), "a contribution was added twice"
                new[p][rc] = have[p][rc] | incoming
            else:
                assert incoming == set(range(n)), "all-gather forwarded an unfinished chunk"
                new[p][rc] = incoming
        have = new
    for p in range(n):
        for c in range(n):
            assert have[p][c] == set(range(n))


@pytest.mark.parametrize("gpn", [1, 2, 4, 8])
def test_tree_chains(gpn):
    for tree in range(gpn):
        chain = schedule.tree_chain(gpn, tree)
        assert sorted(chain) == list(range(gpn))
        assert chain[-1] == tree  # root
    if gpn >= 4:
        # odd trees walk the node the other way round
        assert schedule.tree_chain(gpn, 0)[0] != schedule.tree_chain(gpn, 1)[0] or gpn == 2


def test_split_span_partitions():
    for total, parts in itertools.product([0, 1, 7, 64, 1000, 4097], [1, 2, 3, 8]):
        spans = [schedule.split_span(total, parts, i) for i in range(parts)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
            assert e0 == b1 and b0 <= e0


@pytest.mark.parametrize("tiles_m,tiles_n", [(1, 1), (7, 3), (32, 16), (33, 5), (64, 32), (16, 1)])
@pytest.mark.parametrize("m_fastest,group_m", [(0, 0), (1, 0), (1, 16), (1, 6)])
def test_gemm_tile_order_covers_every_tile_once(tiles_m, tiles_n, m_fastest, group_m):
    """The persistent GEMM's tile order is a bijection onto the tile grid, for
    the single-CTA kernel and (as row-block pairs) for the CTA-pair kernel."""
    from penny_b200.parallel import schedule
    for m_rot in (0, 2 * (tiles_m // 3)):
        total = schedule.gemm_tile_at(tiles_m, tiles_n, 0, m_rot, m_fastest, group_m)[2]
        assert total == tiles_m * tiles_n
        seen = {schedule.gemm_tile_at(tiles_m, tiles_n, t, m_rot, m_fastest, group_m)[:2] for t in range(total)}
        assert seen == {(m, n) for m in range(tiles_m) for n in range(tiles_n)}
        # pairs: CTA 0 and CTA 1 of a pair get vertically adjacent row blocks of the same column block
        ptotal = schedule.gemm_tile_at(tiles_m, tiles_n, 0, m_rot, m_fastest, group_m, pair_rank=0)[2]
        assert ptotal == ((tiles_m + 1) // 2) * tiles_n
        got = set()
        for t in range(ptotal):
            m0, n0, _ = schedule.gemm_tile_at(tiles_m, tiles_n, t, m_rot, m_fastest, group_m, pair_rank=0)
            m1, n1, _ = schedule.gemm_tile_at(tiles_m, tiles_n, t, m_rot, m_fastest, group_m, pair_rank=1)
            assert m0 % 2 == 0 and m1 == m0 + 1 and n0 == n1
            got.add((m0, n0))
            if m1 < tiles_m:
                got.add((m1, n1))
            else:
                assert tiles_m % 2 == 1 and m1 == tiles_m   # the odd last row block has no partner
        assert got == {(m, n) for m in range(tiles_m) for n in range(tiles_n)}


def test_gemm_tile_order_band_is_squareish():
    """With bands of 16 row blocks, the 148 tiles in flight touch 16 row blocks and
    about 10 column blocks instead of all 64 row blocks and 3 columns."""
    from penny_b200.parallel import schedule
    wave = [schedule.gemm_tile_at(64, 32, t, group_m=16)[:2] for t in range(148)]
    assert len({m for m, _ in wave}) == 16 and len({n for _, n in wave}) == 10
    flat = [schedule.gemm_tile_at(64, 32, t, group_m=0)[:2] for t in range(148)]
    assert len({m for m, _ in flat}) == 64 and len({n for _, n in flat}) == 3


@pytest.mark.parametrize("tiles_m,tiles_n,num_kb", [(32, 14, 64), (32, 16, 64), (64, 32, 128), (1, 16, 64), (1, 7, 64),
                                                   (13, 11, 24), (3, 3, 5), (32, 3, 64), (2, 2, 4), (32, 16, 8)])
def test_gemm_split_tail_covers_every_k_step_once(tiles_m, tiles_n, num_kb):
    """Full waves plus the K-split last wave: every (pair tile, K step) is computed by
    exactly one CTA pair, a pair gets at most one split unit and it comes last, and
    the ranges of a split tile are numbered 0..split_s-1."""
    from penny_b200.parallel import schedule
    npairs = 74
    ptiles = ((tiles_m + 1) // 2) * tiles_n
    seen = {}
    segs = {}
    for pair in range(npairs):
        it, had_split = 0, False
        while True:
            w = schedule.gemm_pair_work(tiles_m, tiles_n, npairs, num_kb, pair, it)
            if w is None:
                break
            assert not had_split, "a split unit must be the last unit of its pair"
            if w["split_s"] > 1 and w["tile"] >= w["split_first"]:
                had_split = True
                assert w["kb1"] - w["kb0"] >= 4
                segs.setdefault(w["tile"], []).append(w["seg"])
            else:
                assert (w["kb0"], w["kb1"], w["seg"]) == (0, num_kb, 0)
            for kb in range(w["kb0"], w["kb1"]):
                assert (w["tile"], kb) not in seen
                seen[(w["tile"], kb)] = pair
            it += 1
            assert it < 10000
    assert len(seen) == ptiles * num_kb
    for tile, ss in segs.items():
        assert sorted(ss) == list(range(len(ss))) and len(ss) >= 2


def test_gemm_split_tail_plan_examples():
    from penny_b200.parallel import schedule
    # 224 pair tiles on 74 pairs: three full waves, the two leftover tiles cut 8 ways
    w = schedule.gemm_pair_work(32, 14, 74, 64, 0, 3)
    assert (w["split_first"], w["split_s"], w["tile"], w["kb0"], w["kb1"]) == (222, 8, 222, 0, 8)
    # an exact multiple of the grid is never split
    assert schedule.gemm_pair_work(4, 37, 74, 64, 0, 0)["split_s"] == 1
    # too few K steps for even two ranges of four
    assert schedule.gemm_pair_work(3, 3, 74, 5, 0, 0)["split_s"] == 1


def test_cpp_schedule_properties(tmp_path):
    """The same headers the kernels include, compiled as plain C++ and checked
    exhaustively (rings are Hamiltonian, send/receive chunks pair up, every chunk
    is reduced exactly once, GEMM tile and K-step lists are exact covers)."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    exe = tmp_path / "schedule_test"
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-o", str(exe), os.path.join(root, "tests", "cpp", "schedule_test.cpp")])
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "schedule_test ok" in out.stdout


@pytest.mark.parametrize("num_kb,splits,bt", [(64, 8, 64), (64, 3, 64), (8, 4, 64), (28, 5, 64), (224, 7, 64),
                                              (64, 6, 32), (7, 7, 128), (1, 1, 64), (13, 2, 128)])
def test_decode_gemm_cluster_split(num_kb, splits, bt):
    """Decode GEMM: the K ranges of a cluster cover every K step once and differ by at
    most one step; the column slices of the batch tile cover it once and nobody owns nothing;
    every source has its own slot in every receiver and the receive area is exactly
    what the slots need."""
    from penny_b200.parallel import schedule
    chunk = bt
    plans = [schedule.decode_plan(num_kb, splits, r, bt) for r in range(splits)]
    assert plans[0]["kb0"] == 0 and plans[-1]["kb1"] == num_kb
    sizes = []
    for a, b in zip(plans, plans[1:]):
        assert a["kb1"] == b["kb0"]
    for p in plans:
        assert p["kb1"] > p["kb0"]
        sizes.append(p["kb1"] - p["kb0"])
    assert max(sizes) - min(sizes) <= 1
    sl = plans[0]["slice"]
    owned = []
    for r in range(splits):
        lo, hi = r * sl, min(chunk, (r + 1) * sl)
        assert hi > lo, "a CTA that owns no column would still be waited for"
        owned += list(range(lo, hi))
    assert owned == list(range(chunk))
    for dst in range(splits):
        slots = sorted(schedule.decode_recv_slot(src, dst) for src in range(splits) if src != dst)
        assert slots == list(range(splits - 1))
    want = 0 if splits == 1 else (splits - 1) * sl * 128
    assert plans[0]["recv_floats"] == want


def test_decode_gemm_split_choice_fills_the_gpu():
    """Narrow tensor-parallel shards get enough K ranges to put CTAs on most SMs, all CTAs
    stay resident at once, short K ranges are not split, wide matrices are left alone."""
    from penny_b200.parallel import schedule
    # (tiles, num_kb): TP-8 shards of a Llama-3-8B layer: qkv, o_proj, gate/up, down
    assert schedule.decode_choose_splits(6, 64) == 8
    assert schedule.decode_choose_splits(32, 8) == 1      # 8 K steps: a range of 4 is not worth a cluster
    assert schedule.decode_choose_splits(28, 64) == 8
    assert schedule.decode_choose_splits(32, 28) == 4     # ranges of 7 steps
    for tiles, num_kb in [(6, 64), (28, 64), (32, 28), (48, 64), (32, 64), (32, 224), (126, 64), (24, 64), (112, 64)]:
        s = schedule.decode_choose_splits(tiles, num_kb)
        assert 1 <= s <= 8 and num_kb // s >= 6 and tiles * s <= 2 * 148
    # whole-model matrices: gate/up (224 tiles) and the LM head (1002 tiles) need no split
    assert schedule.decode_choose_splits(224, 64) == 1
    assert schedule.decode_choose_splits(1002, 64) == 1
    assert schedule.decode_choose_splits(32, 224) == 8
    assert schedule.decode_choose_splits(126, 64) == 2
