"""The flag protocol of the symmetric-memory kernels, exercised on the host: random interleavings, a late
rank, back-to-back collectives of different kinds on the same flags, and a rank that never raises its flag."""
import time

import numpy as np
import pytest

from autoparallel_b200.runtime import protocol_model as pm


@pytest.mark.parametrize("n", [2, 4, 8])
def test_all_gather_and_reduce_scatter_interleave_correctly(n):
    m = 16
    rng = np.random.default_rng(0)
    shards = rng.standard_normal((3, n, m)).astype(np.float32)          # [epoch][rank]
    partials = rng.standard_normal((3, n, n * m)).astype(np.float32)    # [epoch][rank] full-size products

    def body(f, r):
        outs, epoch = [], 0
        for e in range(3):  # kernels of one rank run in stream order; epochs grow by one per collective
            epoch += 1
            outs.append(pm.all_gather(f, r, epoch, shards[e, r]))
            epoch += 1
            outs.append(pm.gemm_reduce_scatter(f, r, epoch, partials[e, r]))
        return outs

    f, res = pm.run_ranks(n, body, stage_elems=n * n * m, jitter=2e-4, seed=n)
    assert f.errors == []
    for r in range(n):
        for e in range(3):
            assert np.array_equal(res[r][2 * e], shards[e].reshape(-1))
            want = partials[e].sum(0)[r * m:(r + 1) * m]
            assert np.allclose(res[r][2 * e + 1], want, atol=1e-5)


def test_a_late_rank_is_waited_for():
    n, m = 4, 8
    data = np.arange(n * m, dtype=np.float32).reshape(n, m)

    def body(f, r):
        if r == 3:
            time.sleep(0.15)  # well inside the wait limit
        return pm.all_gather(f, r, 1, data[r])

    f, res = pm.run_ranks(n, body, stage_elems=m, wait_limit_s=1.0)
    assert f.errors == [] and all(np.array_equal(x, data.reshape(-1)) for x in res)


def test_a_flag_that_is_never_raised_ends_in_a_bounded_error():
    n, m = 4, 8
    data = np.ones((n, m), dtype=np.float32)

    def body(f, r):
        return pm.all_gather(f, r, 1, data[r], skip_ready=(r == 2))

    t0 = time.monotonic()
    f, res = pm.run_ranks(n, body, stage_elems=m, wait_limit_s=0.2)
    assert time.monotonic() - t0 < 2.0  # nobody blocks: every wait gives up after its limit
    assert res[2] is not None  # the silent rank itself could pull everything
    assert all(res[r] is None for r in (0, 1, 3))
    assert {(e.rank, e.flag, e.peer, e.expected, e.observed) for e in f.errors} == {(r, "ready", 2, 1, 0) for r in (0, 1, 3)}
    # the next collective cannot start either: the ranks that gave up never said "done", and that is reported too
    f2_errors_before = len(f.errors)
    assert pm.all_gather(f, 2, 2, data[2]) is None and len(f.errors) == f2_errors_before + 1
    assert f.errors[-1].flag == "done" and f.errors[-1].rank == 2


def test_reduce_scatter_waits_for_every_contribution():
    n, m = 2, 4
    partial = np.ones((n, n * m), dtype=np.float32)

    def body(f, r):
        if r == 1:
            return None  # rank 1 never launches its kernel
        return pm.gemm_reduce_scatter(f, r, 1, partial[r])

    f, res = pm.run_ranks(n, body, stage_elems=n * m, wait_limit_s=0.2)
    assert res[0] is None and f.errors and f.errors[0].rank == 0 and f.errors[0].peer == 1


@pytest.mark.parametrize("requests", [0, 3, 100])
def test_dynamic_tiles_are_each_handled_once_even_when_pairs_leave(requests):
    """Tile ring of the CTA-pair GEMM: every tile goes to exactly one pair, all readers of a pair see the same
    sequence, pairs that leave on request never exceed half of the launch, and the counters are back at zero
    for the next launch (which is run right away)."""
    c = pm.TileCounters()
    num_tiles, num_pairs = 97, 8
    for launch in range(2):
        c.request(requests)
        asked = c.requests
        seen = pm.run_dynamic_gemm(c, num_tiles, num_pairs, readers=10, jitter=1e-4, seed=launch)
        tiles = []
        for p in range(num_pairs):
            assert all(s == seen[p][0] for s in seen[p])  # producer, MMA and epilogue roles agree
            tiles += seen[p][0]
        assert sorted(tiles) == list(range(num_tiles))
        idle = sum(1 for p in range(num_pairs) if not seen[p][0])
        assert idle <= max(num_pairs // 2, 0) + 0 or requests == 0
        assert (c.next_tile, c.left, c.yielded) == (0, 0, 0)
        assert c.requests == max(0, asked - num_pairs // 2)  # granted requests are used up, the rest carry over


# ------------------------------------------------------------------------------------- attention pipeline
def _attention_reference(q, k, v, causal, scale):
    import numpy as np

    s = (q @ k.T) * scale
    if causal:
        first = k.shape[0] - q.shape[0]
        s = np.where(np.arange(k.shape[0])[None, :] <= (first + np.arange(q.shape[0]))[:, None], s, -np.inf)
    mx = s.max(1, keepdims=True)
    e = np.exp(s - mx)
    return (e / e.sum(1, keepdims=True)) @ v, np.log(e.sum(1)) + mx[:, 0]


@pytest.mark.parametrize("causal,keys", [(True, 64), (True, 192), (True, 256), (False, 96), (False, 32)])
def test_attention_pipeline_schedule_is_complete_and_exact(causal, keys):
    """Loader, MMA issuer and the two softmax groups of the attention kernel, as host threads with the kernel's
    barriers, three-slot K/V ring and deferred accumulation: every interleaving must give plain attention."""
    import numpy as np

    from autoparallel_b200.runtime.protocol_model import run_attention_pipeline

    rng = np.random.default_rng(keys)
    tile, d = 32, 8
    q = rng.standard_normal((2 * tile, d))
    k = rng.standard_normal((keys, d))
    v = rng.standard_normal((keys, d))
    want, want_lse = _attention_reference(q, k, v, causal, 0.3)
    for seed in range(3):
        out, lse, errors = run_attention_pipeline(q, k, v, causal, 0.3, jitter=0.002, seed=seed, tile=tile)
        assert errors == []
        assert np.abs(out - want).max() < 1e-12 and np.abs(lse - want_lse).max() < 1e-12


@pytest.mark.parametrize("ring", [2, 3, 4])
def test_attention_pipeline_ring_depth_only_changes_prefetch(ring):
    """Two slots are the minimum (V_j and K_{j+1} are live together); more only let the loader run ahead."""
    import numpy as np

    from autoparallel_b200.runtime import protocol_model as pm

    rng = np.random.default_rng(0)
    q, k, v = rng.standard_normal((64, 8)), rng.standard_normal((128, 8)), rng.standard_normal((128, 8))
    out, lse, errors = pm.run_attention_pipeline(q, k, v, True, 1.0, ring=ring, tile=32, jitter=0.001)
    want, _ = _attention_reference(q, k, v, True, 1.0)
    assert errors == [] and np.abs(out - want).max() < 1e-12


def test_swizzle_offsets_are_a_permutation_of_each_atom():
    from autoparallel_b200.runtime.protocol_model import swizzle128_offset

    for atom in range(4):  # an atom is 8 rows x 128 bytes
        seen = {swizzle128_offset(atom * 8 + r, c) for r in range(8) for c in range(8)}
        assert seen == {atom * 1024 + 16 * i for i in range(64)}
    assert swizzle128_offset(0, 3) == 48 and swizzle128_offset(1, 0) == 128 + 16 and swizzle128_offset(9, 1) == 9 * 128
