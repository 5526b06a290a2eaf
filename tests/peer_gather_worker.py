"""Worker of test_peer_gather_multi_gpu.py: one process per GPU, launched by torchrun.

Every rank owns the KV heads of its shard of a small sharded decode and runs it three steps in a row through
PeerHeadGather (merge kernel stores into every GPU's gathered buffer + arrive-and-wait kernel), alternating
the two gathered buffers; after every step the gathered buffer must equal, bit for bit and on every rank, an
NCCL all-gather of the ranks' local outputs, and those must equal a plain single-GPU-style decode of the
shard.  No wait may have run out.  Prints "PEER_GATHER_OK" on rank 0 when all of that held.
"""

import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "rotorquant-vllm_b200"))
sys.path.insert(0, os.path.dirname(HERE))

import gpu_util  # noqa: E402
from oracle import rq_oracle  # noqa: E402  (checker only)
from rotorquant_vllm import cuda as rq  # noqa: E402
from rotorquant_vllm import parallel  # noqa: E402
from rotorquant_vllm import synthetic as syn  # noqa: E402


def main() -> int:
    rank, local, world = (int(os.environ[k]) for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    H, HQ, bs = 8, 32, 16
    kv_lo, kv_hi, q_lo, q_hi = parallel.shard_heads(HQ, H, rank, world)
    h_loc, hq_loc = kv_hi - kv_lo, q_hi - q_lo
    p = gpu_util.params("iso_fast", 3, 3)
    lens = [700, 33, 1, 260]
    seq_lens = torch.tensor(lens, dtype=torch.int32)
    bt, nb = syn.make_block_table(seq_lens, bs, 11)
    slots = syn.slot_mapping_for(bt, seq_lens, bs)
    key, value = syn.make_kv(int(seq_lens.sum()), H, 128, torch.bfloat16, 11)      # same data on every rank
    full = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)
    rq_oracle.compress_and_store(key, value, full, slots, p["R"], p["k_boundaries"], p["v_boundaries"])
    cache = parallel.slice_cache_heads(full, H, kv_lo, kv_hi).to(dev)
    c = {k: v.to(dev) for k, v in dict(bt=bt, sl=seq_lens, ck=p["k_centroids"], cv=p["v_centroids"], R=p["R"]).items()}
    gather = parallel.PeerHeadGather(len(lens), hq_loc, 128, torch.bfloat16, dev)
    ok = True
    for step in range(3):
        q = syn.make_queries(len(lens), HQ, 128, torch.bfloat16, 100 + step)[:, q_lo:q_hi].contiguous().to(dev)
        want = rq.fused_paged_rq_decode(q, cache, c["bt"], c["sl"], c["ck"], c["cv"], c["R"], h_loc, 128, bs)
        g = gather.begin()
        parity = gather.parity
        rq.fused_paged_rq_decode(q, cache, c["bt"], c["sl"], c["ck"], c["cv"], c["R"], h_loc, 128, bs,
                                 out=g.local, peer_out_ptrs=g.peer_ptrs)
        result = gather.finish()                     # (num_seqs, world, heads per rank, 128)
        torch.cuda.synchronize(dev)
        ref = torch.empty(world, *want.shape, dtype=want.dtype, device=dev)
        dist.all_gather_into_tensor(ref.view(-1, *want.shape[1:]), want)
        ok = ok and torch.equal(gather.buffer[parity], ref) and torch.equal(result, ref.permute(1, 0, 2, 3))
        ok = ok and parity == (step & 1)
    ok = ok and not gather.wait_expired()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("PEER_GATHER_OK", flush=True)
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 1 else 1


if __name__ == "__main__":
    sys.exit(main())
