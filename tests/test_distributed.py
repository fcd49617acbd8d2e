"""Host-side sharding logic with two gloo ranks on CPU: column shards of a quantized dense
and KV-head shards of SDPA reproduce the unsharded oracle after the all-gather."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from compute_b200 import distributed as cd
from oracle import oracle as orc
from tests.helpers import qdense_inputs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, K, N, G = 3, 128, 256, 64
        x, w, s, b = qdense_inputs(17, M, K, N, scale_layout="kgroup", group=G)
        full = orc.qdense_linear(x, w, orc.expand_scales(s, "kgroup", K, N, G), None, b, 1, orc.ACT_SILU)
        wl, sl, bl = cd.shard_quantized_dense(w, s, b, "kgroup", G, rank, world)
        part = orc.qdense_linear(x, wl, orc.expand_scales(sl, "kgroup", K, N // world, G), None, bl, 1, orc.ACT_SILU)
        got = cd.all_gather_columns(torch.from_numpy(part)).numpy()
        ok1 = np.array_equal(got, full)            # column-independent op: shards are bit-identical
        # reference scale layout with blocks along N
        x2, w2, s2, b2 = qdense_inputs(18, M, K, N, scale_layout="ref", block_size=32)
        full2 = orc.qdense_linear(x2, w2, s2, None, b2, 32)
        wl2, sl2, bl2 = cd.shard_quantized_dense(w2, s2, b2, "ref", 32, rank, world)
        got2 = cd.all_gather_columns(torch.from_numpy(orc.qdense_linear(x2, wl2, sl2, None, bl2, 32))).numpy()
        ok2 = np.array_equal(got2, full2)
        # SDPA by KV-head groups
        rng = np.random.default_rng(3)
        qq = rng.standard_normal((2, 8, 5, 8), dtype=np.float32)
        kk = rng.standard_normal((2, 4, 6, 8), dtype=np.float32)
        vv = rng.standard_normal((2, 4, 6, 8), dtype=np.float32)
        want = orc.sdpa(qq, kk, vv, causal=False)
        hq, hk = cd.kv_head_shard(8, 4, rank, world)
        mine = torch.from_numpy(orc.sdpa(qq[:, hq], kk[:, hk], vv[:, hk]))
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ok3 = np.array_equal(torch.cat(parts, dim=1).numpy(), want)
        q.put((rank, ok1, ok2, ok3))
    finally:
        dist.destroy_process_group()


def test_two_rank_sharding_matches_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok1, ok2, ok3 in results:
        assert ok1 and ok2 and ok3, (rank, ok1, ok2, ok3)


def test_shard_helpers_reject_bad_splits():
    assert cd.column_shard(14336, 7, 8) == slice(7 * 1792, 14336)
    with pytest.raises(ValueError):
        cd.column_shard(100, 0, 8)
    with pytest.raises(ValueError):
        cd.kv_head_shard(32, 8, 0, 3)
    assert cd.kv_head_shard(32, 8, 1, 4) == (slice(8, 16), slice(2, 4))
