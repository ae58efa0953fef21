"""Multi-rank host logic on CPU: two gloo ranks shard the requests and the column-split
layer exactly as the GPU ranks do; the oracle stands in for the kernels."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from aion_b200 import sharding


def test_request_shard_covers_everything_once():
    for total in (0, 1, 7, 8, 512, 513):
        for world in (1, 2, 3, 8):
            got = []
            for r in range(world):
                s = sharding.request_shard(total, world, r)
                got += list(range(total))[s]
            assert got == list(range(total))
            sizes = [len(range(total)[sharding.request_shard(total, world, r)]) for r in range(world)]
            assert max(sizes) - min(sizes) <= 1


def test_column_shard_multiples():
    assert [sharding.column_shard(28672, 8, r) for r in (0, 7)] == [(0, 3584), (25088, 28672)]
    with pytest.raises(ValueError):
        sharding.column_shard(100, 8, 0)


def _worker(rank: int, world: int, port: int, tmp: str):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import oracle

    m, k, n = 3, 256, 128
    rng = np.random.default_rng(1234)                     # every rank builds the same full problem
    w = (rng.standard_normal((k, n)) * 0.02).astype(np.float32)
    x = rng.standard_normal((m, k)).astype(np.float32)
    full = oracle.quantize(oracle.Q4_0, w, 0)
    n0, n1 = sharding.column_shard(n, world, rank, multiple=32)
    mine = sharding.slice_kmajor_columns(full, k // 32, n, 18, n0, n1)
    # a column slice of the packed weight is the packed weight of the column slice
    assert np.array_equal(mine, oracle.quantize(oracle.Q4_0, w[:, n0:n1], 0))
    y_loc = oracle.matmul_q(oracle.Q4_0, x, mine, m, n1 - n0, k).reshape(m, n1 - n0)
    gather = torch.zeros((world, m, n1 - n0), dtype=torch.float32)
    dist.all_gather_into_tensor(gather.view(-1), torch.from_numpy(y_loc).reshape(-1))
    y = sharding.assemble_gathered(gather.numpy())
    want = oracle.matmul_q(oracle.Q4_0, x, full, m, n, k).reshape(m, n)
    assert np.array_equal(y, want), "column-split + all-gather must reproduce the unsplit result bit for bit"

    # batch sharding: each rank decodes its block of requests; gathering the blocks gives the batch
    total = 6
    sl = sharding.request_shard(total, world, rank)
    xs = rng.standard_normal((total, k)).astype(np.float32)
    part = oracle.matmul_q(oracle.Q4_0, xs[sl], full, sl.stop - sl.start, n, k).reshape(-1, n)
    parts = [torch.zeros((len(range(total)[sharding.request_shard(total, world, r)]), n)) for r in range(world)]
    dist.all_gather(parts, torch.from_numpy(part))
    whole = oracle.matmul_q(oracle.Q4_0, xs, full, total, n, k).reshape(total, n)
    assert np.array_equal(torch.cat(parts).numpy(), whole)
    # the decoder itself: every op is row-wise, so a request decodes to the same tokens in any shard
    from aion_b200.decoder import DecoderConfig
    from oracle.decoder_ref import OracleDecoder

    cfg = DecoderConfig(layers=1, hidden=64, ffn=128, heads=2, kv_heads=1, head_dim=32, vocab=96, ctx=8)
    drng = np.random.default_rng(7)
    wts = {f"l0.{nm}": (drng.standard_normal(shape) * 0.05).astype(np.float32) for nm, shape in cfg.layer_weights().items()}
    wts["head"] = (drng.standard_normal((cfg.hidden, cfg.vocab)) * 0.05).astype(np.float32)
    emb = drng.standard_normal((cfg.vocab, cfg.hidden)).astype(np.float32)
    tokens = np.array([3, 17, 40, 5, 77, 90], np.int32)
    sl = sharding.request_shard(len(tokens), world, rank)
    mine_dec = OracleDecoder(cfg, sl.stop - sl.start, wts, emb)
    full_dec = OracleDecoder(cfg, len(tokens), wts, emb)
    for t in range(3):
        _, lg_mine, nx_mine = mine_dec.step(tokens[sl] + t, np.full(sl.stop - sl.start, t, np.int32))
        _, lg_full, nx_full = full_dec.step(tokens + t, np.full(len(tokens), t, np.int32))
        assert np.array_equal(lg_mine, lg_full[sl]) and np.array_equal(nx_mine, nx_full[sl])
    dist.barrier()
    dist.destroy_process_group()
    open(os.path.join(tmp, f"ok{rank}"), "w").close()


def test_two_ranks_column_split_and_batch_shard(tmp_path):
    import socket

    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(2))
