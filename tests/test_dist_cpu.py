"""World-size-2 gloo checks of the host-side tensor-parallel logic (no GPU): shard ranges, that sharded
partial results recombine to the unsharded oracle result, and the handle-exchange plumbing."""
import os
import sys

import numpy as np
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, HERE)
    from conftest import load_package
    import oracle_binding

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = load_package()
    lib = pkg.load_library()
    orc = oracle_binding.Oracle(os.path.join(ROOT, "oracle", "liboracle.so"))
    P = pkg.plan
    n, k = 96, 512
    w, s, b = pkg.synth_q4(n, k, seed=1)
    x = pkg.f32_to_bf16(np.random.default_rng(3).normal(size=(1, k)).astype(np.float32))
    _, full64 = orc.qgemm(x, w, s, b, want_f64=True)

    # row-parallel: K cut on 64-element group boundaries, partial sums add up to the full product
    r0, rows, c0, cols = pkg.tp.shard_range(lib, P.SHARD_ROW, n, k, rank, world)
    assert (r0, rows) == (0, n) and cols == k // world and c0 == rank * cols and c0 % 64 == 0
    _, part = orc.qgemm(x[:, c0:c0 + cols], w[:, c0 // 8:(c0 + cols) // 8], s[:, c0 // 64:(c0 + cols) // 64],
                        b[:, c0 // 64:(c0 + cols) // 64], want_f64=True)
    t = torch.from_numpy(part.copy())
    dist.all_reduce(t)
    assert np.allclose(t.numpy(), full64, rtol=1e-12, atol=1e-9)

    # column-parallel: output rows cut in contiguous blocks, gathered rows equal the full product
    r0, rows, c0, cols = pkg.tp.shard_range(lib, P.SHARD_COLUMN, n, k, rank, world)
    assert (c0, cols) == (0, k) and rows == n // world and r0 == rank * rows
    mine = orc.qgemm(x, w[r0:r0 + rows], s[r0:r0 + rows], b[r0:r0 + rows])
    pieces = [None] * world
    dist.all_gather_object(pieces, mine.tolist())
    assert np.array_equal(np.concatenate([np.array(p, dtype=np.uint16) for p in pieces], axis=1), orc.qgemm(x, w, s, b))

    # three-section column shard (B|C|x of the short-conv input projection): each rank takes the same channel range of
    # every third, so the gated conv stays rank-local; the ranks' thirds concatenate to the full thirds
    r0, rows, c0, cols = pkg.tp.shard_range(lib, P.SHARD_COLUMN3, n, k, rank, world)
    third = n // 3
    assert (c0, cols) == (0, k) and rows == third // world and r0 == rank * rows
    full = orc.qgemm(x, w, s, b)[0]
    sel = np.concatenate([np.arange(p * third + r0, p * third + r0 + rows) for p in range(3)])
    mine = orc.qgemm(x, w[sel], s[sel], b[sel])[0]
    pieces = [None] * world
    dist.all_gather_object(pieces, mine.tolist())
    for p in range(3):
        got = np.concatenate([np.array(piece, dtype=np.uint16)[p * rows:(p + 1) * rows] for piece in pieces])
        assert np.array_equal(got, full[p * third:(p + 1) * third])

    # vocabulary-sharded argmax: (max, global index) pairs, lowest index wins among equal maxima
    logits = pkg.bf16_to_f32(pkg.f32_to_bf16(np.random.default_rng(4).normal(size=4096).astype(np.float32)))
    logits[[100, 3000]] = 9.0
    shard = 4096 // world
    loc = logits[rank * shard:(rank + 1) * shard]
    pair = (float(loc.max()), int(loc.argmax()) + rank * shard)
    pairs = [None] * world
    dist.all_gather_object(pairs, pair)
    best = min(pairs, key=lambda p: (-p[0], p[1]))
    assert best[1] == 100 == int(np.argmax(logits))

    # handle exchange keeps rank order
    handles = pkg.tp.gather_handles(dist, bytes([rank]) * 64)
    assert [h[0] for h in handles] == list(range(world))

    # indivisible shapes are rejected
    out = (__import__("ctypes").c_int * 4)()
    assert lib.swlm_shard_range(P.SHARD_ROW, n, 64 * 3, rank, world, out) == -1
    q.put(rank)
    dist.destroy_process_group()


def test_two_rank_sharding_recombines():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29641, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert sorted(q.get(timeout=5) for _ in range(2)) == [0, 1]
