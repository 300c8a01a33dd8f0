"""World-size-2 test of the multi-rank host logic on CPU (gloo): every rank takes the contiguous
range of (batch, head) slices that b200attn_shard_ranges gives it, evaluates it independently (the
CPU oracle stands in for the device here: this test is about the partition, not the kernel), and
the gathered result equals the single-process result with no repacking and no data-path collective.
Also covers the timing reduction the benchmark uses (max over ranks)."""
import os
import socket
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, shape, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import __graft_entry__ as ge
    import oracle_lib as ol
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = ge.load_package()
    B, H, Lq, Lk, D = shape
    begin, count = pkg.shard_ranges(B * H, world)
    Q, K, V = ol.make_qkv(B, H, Lq, Lk, D, 7, "uniform")
    sl = slice(begin[rank], begin[rank] + count[rank])
    # a rank's shard is a contiguous slab of the flat [B*H, L, D] tensors
    qs, ks, vs = (np.ascontiguousarray(x.reshape(B * H, -1, D)[sl])[None] for x in (Q, K, V))
    mine = ol.attention(qs, ks, vs, pe=ol.PE_ROPE_HALF)[0] if count[rank] else np.zeros((0, Lq, D), np.float32)
    sizes = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(sizes, torch.tensor([count[rank]], dtype=torch.int64))
    parts = [torch.zeros(int(s.item()), Lq, D) for s in sizes]
    if len({int(s.item()) for s in sizes}) == 1:
        dist.all_gather(parts, torch.from_numpy(mine))
    else:
        for r in range(world):
            buf = torch.from_numpy(mine) if r == rank else parts[r]
            dist.broadcast(buf, src=r)
            parts[r] = buf
    ms = torch.tensor([10.0 + 5.0 * rank], dtype=torch.float64)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        full = ol.attention(Q, K, V, pe=ol.PE_ROPE_HALF).reshape(B * H, Lq, D)
        got = torch.cat(parts).numpy()
        q.put((bool(np.array_equal(got, full)), float(ms.item()), [int(s.item()) for s in sizes]))
    dist.barrier()
    dist.destroy_process_group()


def _run(shape, world=2):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, shape, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return res


def test_two_ranks_even_split():
    same, ms, sizes = _run((2, 4, 8, 12, 16))
    assert same and ms == 15.0 and sizes == [4, 4]


def test_two_ranks_uneven_split():
    same, ms, sizes = _run((1, 5, 6, 6, 8))
    assert same and sizes == [3, 2]
