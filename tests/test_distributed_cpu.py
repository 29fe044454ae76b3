"""CPU: host logic of the two multi-GPU modes on world_size-2 gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT, load_oracle


def test_batch_shard_and_kv_ranges():
    from muzero_b200.distributed import batch_shard, kv_split_ranges
    for total, world in ((64, 8), (64, 3), (5, 8), (160, 4)):
        parts = [batch_shard(total, r, world) for r in range(world)]
        assert parts[0].start == 0 and parts[-1].stop == total
        assert all(a.stop == b.start for a, b in zip(parts, parts[1:]))
        sizes = [p.stop - p.start for p in parts]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        batch_shard(8, 8, 8)
    for total, world, g in ((131072 + 128, 8, 64), (131072 + 131, 4, 128), (300, 2, 64), (100, 4, 64)):
        rs = kv_split_ranges(total, world, g)
        assert rs[0][0] == 0 and rs[-1][1] == total
        assert all(a[1] == b[0] for a, b in zip(rs, rs[1:]))
        assert all((e - s) % g == 0 for s, e in rs[:-1])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, q_out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import sys
    sys.path.insert(0, ROOT)
    orc = load_oracle()
    from muzero_b200.distributed import kv_split_decode_attention, kv_split_ranges, batch_shard, pack_partial, unpack_partials
    k, v, q = orc.synth_kv(2, 2, 512, 64, 8, seed=5)           # same on every rank
    s, e = kv_split_ranges(512, world, 64)[rank]

    def record_fn(layer, query, scaling):                        # CPU stand-in for the CUDA partial kernel
        return pack_partial(*orc.attention_partial_oracle(query, layer[0], layer[1], scaling, 4))

    def merge_fn(records, dtype):                                # ... and for the merge kernel
        ms, ls, accs = unpack_partials(records)
        out = orc.lse_merge_oracle(list(ms), list(ls), list(accs))
        return out.unsqueeze(1).to(dtype)

    out = kv_split_decode_attention((k[:, :, s:e].float(), v[:, :, s:e].float()), q, 0.125, out_dtype=torch.float32,
                                    record_fn=record_fn, merge_fn=merge_fn)
    m, l, acc = orc.attention_partial_oracle(q, k.float(), v.float(), 0.125, 4)
    whole = (acc / l.unsqueeze(-1)).unsqueeze(1)
    err = (out - whole).abs().max().item()
    # batch sharding: each rank's slice of a batched result equals the unsharded result's rows
    sl = batch_shard(2, rank, world)
    mb, lb, ab = orc.attention_partial_oracle(q[sl], k[sl].float(), v[sl].float(), 0.125, 4)
    err_b = ((ab / lb.unsqueeze(-1)) - (acc / l.unsqueeze(-1))[sl]).abs().max().item()
    q_out.put((rank, err, err_b))
    dist.destroy_process_group()


def test_kv_split_and_batch_shard_world2():
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, err_b in results:
        assert err < 1e-5 and err_b < 1e-6, (rank, err, err_b)
