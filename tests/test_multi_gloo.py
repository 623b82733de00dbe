"""The multi-rank path on CPU (gloo, world_size 2): minibatch sharding and the weight-gradient
all-reduce reproduce the single-rank result. The device kernels are replaced by the oracle here;
what is under test is the host-side decomposition that bench.py --gpus N relies on:
fprop/bprop shard over N with no exchange, update sums fp32 partial gradients over ranks."""
import os
import socket
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist        # noqa: E402
import torch.multiprocessing as mp      # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from nervanagpu_b200.convnet import bucket_layout, shard_minibatch
    from oracle import reference_math as rm
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    try:
        full = rm.ConvDims(32, 4, 8, 1, 6, 6, 1, 3, 3, 0, 1, 1, 1, 1, 1)
        rng = np.random.default_rng(7)                      # same data on every rank
        I = rng.uniform(0, 1, full.dimI).astype(np.float16)
        F = rng.normal(0, 0.1, full.dimF).astype(np.float16)
        E = rng.uniform(-1, 1, full.dimO).astype(np.float16)
        I_r, E_r = shard_minibatch(I, rank, world), shard_minibatch(E, rank, world)
        local = rm.ConvDims(32 // world, 4, 8, 1, 6, 6, 1, 3, 3, 0, 1, 1, 1, 1, 1)
        # forward / backward: no exchange, each rank owns its images
        O_r = rm.conv_fprop(local, I_r, F)
        gI_r = rm.conv_bprop(local, F, E_r)
        # update: partial gradient on the shard, fp32 all-reduce over a flat two-layer bucket
        sizes = [int(np.prod(full.dimF)), 24]
        offsets, total = bucket_layout(sizes)
        bucket = np.zeros(total, dtype=np.float32)
        bucket[offsets[0]:offsets[0] + sizes[0]] = rm.conv_update(local, I_r, E_r).ravel()
        bucket[offsets[1]:offsets[1] + sizes[1]] = rank + 1.0
        t = torch.from_numpy(bucket)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        np.savez(os.path.join(out_dir, "rank%d.npz" % rank), O=O_r, gI=gI_r, bucket=bucket)
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_sharded_conv_matches_single_rank(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)

    sys.path.insert(0, ROOT)
    from nervanagpu_b200.convnet import bucket_layout
    from oracle import reference_math as rm
    full = rm.ConvDims(32, 4, 8, 1, 6, 6, 1, 3, 3, 0, 1, 1, 1, 1, 1)
    rng = np.random.default_rng(7)
    I = rng.uniform(0, 1, full.dimI).astype(np.float16)
    F = rng.normal(0, 0.1, full.dimF).astype(np.float16)
    E = rng.uniform(-1, 1, full.dimO).astype(np.float16)
    O, gI, gF = rm.conv_fprop(full, I, F), rm.conv_bprop(full, F, E), rm.conv_update(full, I, E)
    parts = [np.load(os.path.join(str(tmp_path), "rank%d.npz" % r)) for r in range(world)]
    assert np.array_equal(np.concatenate([p["O"] for p in parts], axis=-1), O)
    np.testing.assert_allclose(np.concatenate([p["gI"] for p in parts], axis=-1), gI, rtol=0, atol=1e-5)
    sizes = [int(np.prod(full.dimF)), 24]
    offsets, total = bucket_layout(sizes)
    for p in parts:                                   # every rank holds the same reduced bucket
        got = p["bucket"]
        np.testing.assert_allclose(got[offsets[0]:offsets[0] + sizes[0]].reshape(full.dimF), gF, rtol=1e-5, atol=1e-4)
        assert (got[offsets[1]:offsets[1] + sizes[1]] == 3.0).all()
        assert (got[offsets[0] + sizes[0]:offsets[1]] == 0).all()       # alignment padding stays zero


def test_shard_and_bucket_helpers():
    from nervanagpu_b200.convnet import bucket_layout, shard_minibatch
    x = np.arange(2 * 3 * 32).reshape(2, 3, 32)
    a, b = shard_minibatch(x, 0, 2), shard_minibatch(x, 1, 2)
    assert a.shape == (2, 3, 16) and a.flags["C_CONTIGUOUS"]
    assert np.array_equal(np.concatenate([a, b], axis=-1), x)
    with pytest.raises(ValueError):
        shard_minibatch(x, 0, 8)        # 4 images per rank: not a multiple of 8
    with pytest.raises(ValueError):
        shard_minibatch(x, 0, 3)
    offsets, total = bucket_layout([23232, 5, 8])
    assert offsets == [0, 23232, 23240] and total == 23248


def test_gradient_buckets_cover_every_layer_once_in_completion_order():
    from nervanagpu_b200.convnet import comm_bucket_order
    alexnet = [23232, 307200, 663552, 884736, 589824]
    vgg_a = [1728, 73728, 294912, 589824, 1179648, 2359296, 2359296, 2359296]
    for sizes, want in ((alexnet, [(2, 5), (1, 2), (0, 1)]),
                        (vgg_a, [(4, 8), (3, 4), (2, 3), (1, 2), (0, 1)]),
                        ([7], [(0, 1)]), ([5, 5], [(1, 2), (0, 1)])):
        got = comm_bucket_order(sizes)
        assert got == want
        covered = sorted(i for first, last in got for i in range(first, last))
        assert covered == list(range(len(sizes)))
        assert [b[0] for b in got] == sorted((b[0] for b in got), reverse=True)   # top of the stack first
