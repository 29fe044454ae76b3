"""GPU (needs 2 devices, skipped otherwise): KV-sequence split over NCCL and batch sharding.

Each rank holds a contiguous slice of one long sequence in its own quantized store, computes the
partial (m, l, acc) triple of its slice, the triples are all-gathered and merged locally.  The
result on every rank must equal the one-GPU result over the whole sequence."""
import os
import socket

import pytest
import torch

from conftest import ROOT, load_oracle

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, q_out):
    import sys
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import muzero_b200 as mz
    from muzero_b200.cache.attention import decode_attention
    from muzero_b200.distributed import batch_shard, kv_split_decode_attention, kv_split_ranges
    orc = load_oracle()
    B, KVH, H, S, D, bits, G = 2, 2, 8, 4096, 128, 2, 64
    k, v, q = orc.synth_kv(B, KVH, S, D, H, seed=17)
    a, b = kv_split_ranges(S, world, G)[rank]
    # the last rank keeps a residual window, the others hold fully quantized slices
    res = 128 if rank == world - 1 else 0
    mine = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=G, residual_length=res, alpha_key=2.0, alpha_value=2.0))
    mine.update(k[:, :, a:b].cuda().contiguous(), v[:, :, a:b].cuda().contiguous(), {"materialize_full_kv": False})
    out = kv_split_decode_attention(mine, q.cuda(), D ** -0.5, out_dtype=torch.float32)
    # one-GPU result over the whole sequence with the same quantization boundaries
    whole = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=G, residual_length=128, alpha_key=2.0, alpha_value=2.0))
    whole.update(k.cuda(), v.cuda(), {"materialize_full_kv": False})
    ref = decode_attention(whole, q.cuda(), D ** -0.5, out_dtype=torch.float32)
    err = (out - ref).abs().max().item()
    # batch sharding: this rank's slice of the batch equals the same rows of the full-batch result
    sl = batch_shard(B, rank, world)
    part = mz.MuZeroCacheLayer(mz.MuZeroConfig(bits=bits, q_group_size=G, residual_length=128, alpha_key=2.0, alpha_value=2.0))
    part.update(k[sl].cuda().contiguous(), v[sl].cuda().contiguous(), {"materialize_full_kv": False})
    err_b = (decode_attention(part, q[sl].cuda(), D ** -0.5, out_dtype=torch.float32) - ref[sl]).abs().max().item()
    torch.cuda.synchronize()
    q_out.put((rank, err, err_b))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_kv_split_over_nccl_matches_single_gpu():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q_out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q_out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q_out.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for rank, err, err_b in results:
        assert err < 5e-4, (rank, err)        # same codes; the ranges differ, so fp16 operand rounding differs
        assert err_b < 5e-4, (rank, err_b)    # sequences are independent; a smaller batch is cut into other per-warp ranges
