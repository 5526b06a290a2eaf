"""GPU parity at the benchmark configurations' own launch shapes.

The fresh-case tests use small batches; these build the very jobs ``bench.py`` times (same class,
same seeds) -- the CPU-runnable configuration with its aliased block tables, 64 x 4096 (llama-8B
shape), 256 ragged sequences with planar K4/V3 (qwen-7B shape) and one KV head of 8 x 131072 tokens
(the shard one GPU holds of the 70B-shaped long-context configuration at 8 GPUs) -- run the decode
launch exactly as benchmarked and compare sampled output rows with the CPU oracle.
"""

import hashlib

import numpy as np
import pytest
import torch

import gpu_util
import helpers
from gpu_util import DEV
from oracle import tolerance
from rotorquant_vllm import synthetic as syn

pytestmark = pytest.mark.gpu


def test_cpu_roundtrip_configuration_against_the_reference_digest():
    """Configuration 1: fp32 K/V of 2048 tokens, 8 KV heads, iso-fast 3-bit; batch-4 decode with
    32 query heads over block tables that alias the same physical blocks in different orders.
    Cache bytes must hash to the reference's digest and the decode must match the reference's
    committed outputs."""
    from rotorquant_vllm import cuda as rq

    z = np.load(helpers.GOLDEN + "/case_cpu_roundtrip_digest.npz")
    p = gpu_util.params("iso_fast", 3, 3)
    w = syn.WORKLOADS["cpu_roundtrip"]
    key, value = syn.make_kv(w.ctx_max, w.num_kv_heads, 128, w.dtype, 0)

    def sha(t):
        return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()

    if sha(key) != str(z["key_sha"]):
        pytest.skip("torch CPU generator stream differs from the one the digest was made with")
    cache = torch.zeros(w.ctx_max // 16, 16, 2048, dtype=torch.uint8, device=DEV)
    rq.compress_and_store(key.to(DEV), value.to(DEV), cache, torch.arange(w.ctx_max, device=DEV), p["R"].to(DEV),
                          p["k_boundaries"].to(DEV), p["v_boundaries"].to(DEV))
    assert sha(cache.cpu()) == str(z["cache_sha"]), "compressed cache differs from the reference's"
    q = syn.make_queries(w.batch, w.num_q_heads, 128, torch.bfloat16, 0)
    bt = torch.from_numpy(z["block_table"].copy())
    sl = torch.full((w.batch,), w.ctx_max, dtype=torch.int32)
    out = rq.fused_paged_rq_decode(q.to(DEV), cache, bt.to(DEV), sl.to(DEV), p["k_centroids"].to(DEV),
                                   p["v_centroids"].to(DEV), p["R"].to(DEV), 8, 128, 16).cpu()
    ref_out = helpers.from_bits(z["out"], torch.bfloat16)
    ref_rot = torch.from_numpy(z["o_rot"].copy())
    worst, over = tolerance.excess(out, ref_rot, ref_out, torch.bfloat16)
    assert over == 0, f"max diff {worst:.3e}, {over} elements over tolerance"


@pytest.mark.parametrize("workload,world,sample", [
    ("decode_llama8b", 1, 4),            # configuration 2: batch 64, context 4096
    ("decode_qwen7b_planar", 1, 4),      # configuration 3: 256 ragged sequences, planar K4 / V3, G = 7
    ("decode_70b_long", 8, 2),           # configuration 5: the shard of one of 8 GPUs (1 KV head, 8 x 131072)
])
def test_benchmarked_launch_matches_the_oracle(workload, world, sample):
    import bench

    dev = torch.device(DEV)
    torch.cuda.set_device(dev)
    job = bench.GpuJob(syn.WORKLOADS[workload], 0, world, dev)
    job.step()                               # compress-on-write of the step's tokens, then decode
    res = job.parity_check(sample)
    assert res["rows"] == sample * job.HQ
    assert res["over_tolerance"] == 0, res
    assert not bool(torch.isnan(job.out.float()).any())
    # the same launch inside a CUDA graph, as the benchmark replays it
    want = job.out.clone()
    graph = torch.cuda.CUDAGraph()
    job.out.zero_()
    with torch.cuda.graph(graph):
        job.step()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(job.out, want), "graph replay differs from the direct launch"
