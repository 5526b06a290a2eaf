"""Benchmark of the RotorQuant KV-cache hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one attention-layer decode call of the serving path on one batch: compress-on-write
of the step's new K/V tokens into the paged cache, then fused paged decode attention over the
whole compressed context (query rotation, split-KV merge and output rotation included).

* default arm: the CUDA library through its C ABI, one process per GPU (torchrun for N > 1).
  ``value`` is device-resident throughput (inputs already in HBM), ``e2e`` the same step driven
  from pinned HOST buffers with the host<->device copies inside the timed region.
* ``--impl reference``: the reference's CPU path (PyTorch ops, restated in ``oracle/``) on the
  host cores, on a bounded sample of the same workload.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
for _p in (REPO, os.path.join(REPO, "rotorquant-vllm_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

from rotorquant_vllm import parallel  # noqa: E402
from rotorquant_vllm import synthetic as syn  # noqa: E402
from rotorquant_vllm.quantization import IsoQuantMSE, PlanarQuantMSE  # noqa: E402
from rotorquant_vllm.vllm.rotation import build_rotation_matrix  # noqa: E402

METRIC = "fused_paged_decode_tokens_per_s"
UNIT = "tokens/s"
# DRAM bytes per launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum of
# decode_split_kernel) divided by the algorithmic bytes of the same launch; see
# profiles/decode_split_kernel_llama8b.md.  Used to scale `roofline.traffic` to this run's launch.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 155.8e6 / 143.2e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="decode_llama8b",
                    choices=["decode_llama8b", "decode_qwen7b_planar", "decode_70b_long", "prefill_int8"])
    ap.add_argument("--batch", type=int, default=0,
                    help="override the workload's number of sequences (small cases for profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--fused-prefill", action="store_true",
                    help="prefill workload: the single fused kernel instead of stage + attention")
    return ap.parse_args()


# --------------------------------------------------------------------------------------------
# Shared set-up
# --------------------------------------------------------------------------------------------

def make_quantizers(w: syn.Workload):
    def make(bits):
        if w.rq_mode == "iso":
            return IsoQuantMSE(w.head_dim, bits, seed=42, mode=w.iso_mode)
        return PlanarQuantMSE(w.head_dim, bits, seed=42)
    kq = make(w.k_bits)
    vq = kq if w.v_bits == w.k_bits else make(w.v_bits)
    return kq, vq, build_rotation_matrix(kq, w.head_dim, "cpu")


def peaks() -> tuple[float, str]:
    """Measured HBM copy bandwidth of this pool's B200s in GB/s, else the stated fallback."""
    path = os.path.join(REPO, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, "fallback"


def decode_algorithmic_bytes(seq_lens, num_kv_heads: int, num_q_heads: int, block_size: int) -> int:
    """KV payload read once per KV head (136 B per token and head), block-table entries, Q in, O out."""
    total = 0
    for n in seq_lens:
        total += n * num_kv_heads * 136 + ((n + block_size - 1) // block_size) * 4
    total += 2 * len(seq_lens) * num_q_heads * 128 * 2
    return total


class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU while a region runs (read-only
    NVML queries from a thread every few milliseconds; nvidia-smi as a fallback)."""

    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
               "sw_power_cap": 0x4}

    def __init__(self, index: int):
        self.index = index
        self.sm: list[float] = []
        self.bits = 0
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None

    def _visible_index(self) -> int:
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.index])
            except (ValueError, IndexError):
                pass
        return self.index

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self._visible_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
        self._thread = threading.Thread(target=self._poll, daemon=True)
        self._thread.start()

    def _sample(self):
        if self._nvml is not None:
            n = self._nvml
            self.sm.append(float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
            try:
                self.bits |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
            except Exception:
                self.bits |= int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
        else:
            out = subprocess.run(
                ["nvidia-smi", "-i", str(self._visible_index()),
                 "--query-gpu=clocks.sm,clocks.max.sm,clocks_event_reasons.active",
                 "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
            parts = [x.strip() for x in out.split(",")]
            self.sm.append(float(parts[0]))
            self.max_mhz = float(parts[1])
            self.bits |= int(parts[2], 16)

    def _poll(self):
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception:
                pass
            self._stop.wait(0.004)

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        reasons = sorted(name for name, bit in self.REASONS.items() if self.bits & bit)
        return {"sm_mhz": statistics.median(self.sm) if self.sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": reasons, "samples": len(self.sm)}


# --------------------------------------------------------------------------------------------
# The reference's CPU path on a bounded sample (cpu_baseline leg and --impl reference)
# --------------------------------------------------------------------------------------------

class CpuSample:
    """`sample_seqs` sequences of the workload, cache built and stepped with the CPU oracle."""

    def __init__(self, w: syn.Workload, sample_seqs: int, seed: int = 0):
        from oracle import rq_oracle  # the only place bench.py touches oracle/

        self.oracle = rq_oracle
        self.w = w
        self.kq, self.vq, self.R = make_quantizers(w)
        self.seq_lens = syn.make_seq_lens(w.batch, w.ctx_min, w.ctx_max, seed)[:sample_seqs].contiguous()
        s = len(self.seq_lens)
        self.bt, nb = syn.make_block_table(self.seq_lens, w.block_size, seed)
        slots = syn.slot_mapping_for(self.bt, self.seq_lens, w.block_size)
        key, value = syn.make_kv(int(self.seq_lens.sum()), w.num_kv_heads, w.head_dim, w.dtype, seed)
        self.cache = torch.zeros(nb, w.block_size, w.num_kv_heads * 256, dtype=torch.uint8)
        rq_oracle.compress_and_store(key, value, self.cache, slots, self.R, self.kq.boundaries,
                                     self.vq.boundaries)
        # the step's new token of every sampled sequence sits at its last position
        ends = torch.cumsum(self.seq_lens.long(), 0) - 1
        self.new_k, self.new_v, self.new_slots = key[ends].clone(), value[ends].clone(), slots[ends].clone()
        self.q = syn.make_queries(s, w.num_q_heads, w.head_dim, w.dtype, seed)

    def step(self) -> torch.Tensor:
        w, o = self.w, self.oracle
        o.compress_and_store(self.new_k, self.new_v, self.cache, self.new_slots, self.R,
                             self.kq.boundaries, self.vq.boundaries)
        return o.decode(self.q, self.cache, self.bt, self.seq_lens, self.kq.centroids,
                        self.vq.centroids, self.R, w.num_kv_heads, w.head_dim, w.block_size)

    def describe(self) -> str:
        w = self.w
        return (f"{len(self.seq_lens)} of {w.batch} sequences of {w.name} "
                f"(context {int(self.seq_lens.min())}-{int(self.seq_lens.max())}, {w.num_q_heads} query / "
                f"{w.num_kv_heads} KV heads), compress-on-write + decompress + SDPA per step")


def time_cpu_sample(sample: CpuSample, steps: int, warmup: int) -> float:
    """Seconds per step of the CPU path on the sample."""
    for _ in range(warmup):
        sample.step()
    t0 = time.perf_counter()
    for _ in range(steps):
        sample.step()
    return (time.perf_counter() - t0) / steps


def cpu_baseline(w: syn.Workload, budget_s: float = 12.0) -> dict:
    """Oracle port of the reference CPU path, timed on this host within ~budget_s seconds."""
    s = min(4, w.batch)
    sample = CpuSample(w, s)
    per_step = time_cpu_sample(sample, 1, 1)
    steps = max(2, min(50, int(budget_s / max(per_step, 1e-3))))
    per_step = time_cpu_sample(sample, steps, 0)
    return {"value": len(sample.seq_lens) / per_step, "unit": UNIT, "cores": torch.get_num_threads(),
            "kind": "port", "sample": sample.describe() + f", {steps} steps"}


def run_reference_arm(args, w: syn.Workload) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = CpuSample(w, min(4, w.batch))
    steps = max(1, min(args.steps, 40))
    warm = max(1, min(args.warmup, 3))
    per_step = time_cpu_sample(sample, steps, warm)
    n = len(sample.seq_lens)
    value = n / per_step
    base = {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": sample.describe()}
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, 1, w.batch), "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def workload_config(w: syn.Workload, world: int, seqs_per_rank: int, sharding: str = "by sequence",
                    step: str = "compress-on-write of one new token per sequence + fused paged decode") -> dict:
    return {
        "workload": w.name, "num_seqs": seqs_per_rank * (world if sharding == "by sequence" else 1),
        "context": w.ctx_max if w.ctx_min == w.ctx_max else f"{w.ctx_min}-{w.ctx_max}",
        "q_heads": w.num_q_heads, "kv_heads": w.num_kv_heads, "head_dim": w.head_dim,
        "block_size": w.block_size,
        "rq": f"{w.rq_mode}-{w.iso_mode if w.rq_mode == 'iso' else 'givens'} k{w.k_bits} v{w.v_bits}",
        "sharding": sharding,
        "step": step,
        "l2": "compressed cache per GPU is larger than the 126 MB L2",
    }


# --------------------------------------------------------------------------------------------
# The B200 arm
# --------------------------------------------------------------------------------------------

class GpuJob:
    """This rank's share of the workload, resident in HBM, plus the step that runs on it."""

    def __init__(self, w: syn.Workload, rank: int, world: int, device: torch.device):
        from rotorquant_vllm import cuda as rq

        self.rq, self.w, self.dev = rq, w, device
        kq, vq, R = make_quantizers(w)
        self.R = R.to(device)
        self.kc, self.vc = kq.centroids.to(device), vq.centroids.to(device)
        self.kb, self.vb = kq.boundaries.to(device), vq.boundaries.to(device)

        if w.name == "decode_70b_long":
            # one request spans the GPUs: shard by KV head, every rank sees every sequence
            if w.num_kv_heads % world:
                raise SystemExit(f"{w.name}: {w.num_kv_heads} KV heads do not split over {world} GPUs")
            self.sharding = "by KV head"
            self.H = w.num_kv_heads // world
            self.HQ = w.num_q_heads // world
            seed = 0
        else:
            self.sharding = "by sequence"
            self.H, self.HQ = w.num_kv_heads, w.num_q_heads
            seed = rank
        self.seq_lens_host = syn.make_seq_lens(w.batch, w.ctx_min, w.ctx_max, seed)
        B, bs = w.batch, w.block_size
        need = (self.seq_lens_host.long() + bs - 1) // bs
        nblk = int(need.sum())
        gen = torch.Generator(device=device).manual_seed(1000 + rank)
        perm = torch.randperm(nblk, device=device, generator=gen).to(torch.int32)
        self.bt = torch.zeros(B, int(need.max()), dtype=torch.int32, device=device)
        self.cache = torch.zeros(nblk, bs, self.H * 256, dtype=torch.uint8, device=device)
        self.new_k = torch.empty(B, self.H, w.head_dim, dtype=w.dtype, device=device)
        self.new_v = torch.empty_like(self.new_k)
        self.new_slots = torch.empty(B, dtype=torch.int64, device=device)
        ch = 3   # the x10 outlier channel
        pos0 = 0
        for s in range(B):
            n, nb = int(self.seq_lens_host[s]), int(need[s])
            self.bt[s, :nb] = perm[pos0:pos0 + nb]
            pos0 += nb
            pos = torch.arange(n, device=device)
            slots = self.bt[s].long()[pos // bs] * bs + pos % bs
            for lo in range(0, n, 16384):           # bounded temporaries for the long contexts
                hi = min(n, lo + 16384)
                k = torch.randn(hi - lo, self.H, w.head_dim, device=device, generator=gen)
                v = torch.randn(hi - lo, self.H, w.head_dim, device=device, generator=gen)
                k[..., ch] *= 10
                v[..., ch] *= 10
                k, v = k.to(w.dtype), v.to(w.dtype)
                rq.compress_and_store(k, v, self.cache, slots[lo:hi], self.R, self.kb, self.vb)
            self.new_k[s], self.new_v[s], self.new_slots[s] = k[-1], v[-1], slots[-1]
        self.q = torch.randn(B, self.HQ, w.head_dim, device=device, generator=gen).to(w.dtype)
        self.seq_lens = self.seq_lens_host.to(device)
        self.out = torch.empty_like(self.q)
        self.max_seq_len = int(self.seq_lens_host.max())
        self.gathered = None
        if self.sharding == "by KV head" and world > 1:
            self.gathered = torch.empty(B, w.num_q_heads, w.head_dim, dtype=w.dtype, device=device)
        torch.cuda.synchronize(device)

    # one step on device-resident inputs: 4 kernel launches (compress+store, decode plan, stream, merge)
    def step(self):
        w = self.w
        self.rq.compress_and_store(self.new_k, self.new_v, self.cache, self.new_slots, self.R,
                                   self.kb, self.vb)
        self.decode_only()

    def decode_only(self):
        w = self.w
        self.rq.fused_paged_rq_decode(self.q, self.cache, self.bt, self.seq_lens, self.kc, self.vc,
                                      self.R, self.H, w.head_dim, w.block_size, out=self.out,
                                      max_seq_len=self.max_seq_len)

    def gather_heads(self):
        if self.gathered is not None:
            self.gathered = parallel.gather_head_outputs(self.out)

    def algorithmic_bytes(self) -> int:
        return decode_algorithmic_bytes(self.seq_lens_host.tolist(), self.H, self.HQ, self.w.block_size)


def timed(fn, steps: int, device) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the current stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1)


def run_gpu_arm(args, w: syn.Workload) -> None:
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200 arm has no CPU fallback")
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist = torch.distributed
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    job = GpuJob(w, rank, world, device)
    full_step = (lambda: (job.step(), job.gather_heads())) if job.gathered is not None else job.step

    # ---- device-resident throughput: W warm-up steps, then exactly K timed steps ----
    for _ in range(max(args.warmup, 3)):
        full_step()
    graph = None
    if not args.no_graph and job.gathered is None:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                job.step()
            for _ in range(3):
                graph.replay()
        except Exception as exc:  # capture is an optimisation of the launch path only
            print(f"[bench] CUDA graph capture unavailable ({exc}); launching directly", file=sys.stderr)
            graph = None
            torch.cuda.synchronize(device)
    runner = graph.replay if graph is not None else full_step
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    if sampler:
        sampler.start()
    ms_total = timed(runner, args.steps, device)
    barrier()

    # ---- the dominant kernel alone (decode split + merge), same inputs, events per launch ----
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(args.steps)]
    torch.cuda.synchronize(device)
    for a, b in evs:
        job.rq.compress_and_store(job.new_k, job.new_v, job.cache, job.new_slots, job.R, job.kb, job.vb)
        a.record()
        job.decode_only()
        b.record()
    torch.cuda.synchronize(device)
    decode_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    compress_ms = timed(lambda: job.rq.compress_and_store(job.new_k, job.new_v, job.cache, job.new_slots,
                                                          job.R, job.kb, job.vb), args.steps, device) / args.steps
    clocks = sampler.stop() if sampler else None

    # ---- end to end from pinned host buffers ----
    host = {name: getattr(job, name).cpu().pin_memory()
            for name in ("q", "new_k", "new_v", "new_slots", "bt", "seq_lens")}
    out_host = torch.empty(job.out.shape, dtype=job.out.dtype).pin_memory()

    def e2e_step():
        for name, h in host.items():
            getattr(job, name).copy_(h, non_blocking=True)
        job.step()
        job.gather_heads()
        out_host.copy_(job.out, non_blocking=True)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_ms = timed(e2e_step, args.steps, device)
    barrier()
    h2d = sum(h.numel() * h.element_size() for h in host.values())
    d2h = out_host.numel() * out_host.element_size()

    # ---- max over ranks ----
    t = torch.tensor([ms_total, e2e_ms, decode_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, decode_ms = t.tolist()

    if rank == 0:
        seqs_per_step = w.batch * (world if job.sharding == "by sequence" else 1)
        ms_per_step = ms_total / args.steps
        peak, peak_kind = peaks()
        alg = job.algorithmic_bytes()
        achieved = alg / (decode_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": seqs_per_step / (ms_per_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak" if job.sharding == "by sequence" else "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, world, w.batch, job.sharding),
            "clocks": clocks, "cuda_graph": graph is not None,
            "e2e": {"value": seqs_per_step / (e2e_ms / args.steps * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": 4 * args.steps,
            "roofline": {"bound": "hbm", "kernel": "decode_umma_kernel (+ plan and merge kernels)",
                         "achieved": achieved, "peak": peak, "peak_kind": f"{peak_kind} copy bandwidth",
                         "unit": "GB/s", "frac": achieved / peak,
                         "algorithmic_bytes": alg, "kernel_ms": decode_ms,
                         "traffic": alg * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE},
            "decode_tokens_per_s_per_gpu": w.batch / (decode_ms * 1e-3),
            "compress_mtok_per_s_at_decode_batch": w.batch / (compress_ms * 1e-3) / 1e6,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------------
# Prefill workload (secondary metric): compress-on-write of all prompt tokens + INT8 prefill
# --------------------------------------------------------------------------------------------

PREFILL_STEP = "compress-on-write of all prompt tokens + causal INT8 prefill attention over the cache"


def run_prefill_arm(args, w: syn.Workload) -> None:
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    T, B, H, HQ, D, bs = w.ctx_max, w.batch, w.num_kv_heads, w.num_q_heads, w.head_dim, w.block_size
    ops = 4 * D * B * HQ * T * (T + 1) // 2          # causal, QK^T + PV, 2 per multiply-add
    if args.impl == "reference":
        if rank != 0:
            return
        from oracle import rq_oracle

        kq, vq, R = make_quantizers(w)
        seq_lens = torch.tensor([T], dtype=torch.int32)
        bt, nb = syn.make_block_table(seq_lens, bs, 0)
        slots = syn.slot_mapping_for(bt, seq_lens, bs)
        key, value = syn.make_kv(T, H, D, w.dtype, 0)
        q = syn.make_queries(T, HQ, D, w.dtype, 0)
        cache = torch.zeros(nb, bs, H * 256, dtype=torch.uint8)

        def step():
            rq_oracle.compress_and_store(key, value, cache, slots, R, kq.boundaries, vq.boundaries)
            return rq_oracle.prefill(q, cache, bt, seq_lens, kq.centroids, vq.centroids, R, H, D, bs)

        steps = max(1, min(args.steps, 5))
        step()
        t0 = time.perf_counter()
        for _ in range(steps):
            step()
        per = (time.perf_counter() - t0) / steps
        base = {"value": T / per, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                "sample": f"1 of {B} sequences of {T} tokens, compress + decompress + causal SDPA"}
        print(json.dumps({"impl": "reference", "metric": "int8_prefill_tokens_per_s", "value": T / per,
                          "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": 1,
                          "ms_per_step": per * 1e3, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": workload_config(w, 1, B, step=PREFILL_STEP), "cpu_baseline": base, "gpu_launches": 0,
                          "e2e": {"value": T / per, "unit": UNIT, "h2d_bytes_per_step": 0,
                                  "d2h_bytes_per_step": 0}}))
        return

    from rotorquant_vllm import cuda as rq

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=device)
    kq, vq, R = make_quantizers(w)
    R = R.to(device)
    kc, vc, kb, vb = (t.to(device) for t in (kq.centroids, vq.centroids, kq.boundaries, vq.boundaries))
    gen = torch.Generator(device=device).manual_seed(rank)
    nblk = B * T // bs
    cache = torch.zeros(nblk, bs, H * 256, dtype=torch.uint8, device=device)
    bt = torch.randperm(nblk, device=device, generator=gen).to(torch.int32).reshape(B, T // bs).contiguous()
    pos = torch.arange(T, device=device)
    slots = torch.cat([bt[s].long()[pos // bs] * bs + pos % bs for s in range(B)])
    key = torch.randn(B * T, H, D, device=device, generator=gen)
    value = torch.randn(B * T, H, D, device=device, generator=gen)
    key[..., 3] *= 10
    value[..., 3] *= 10
    key, value = key.to(w.dtype), value.to(w.dtype)
    q = torch.randn(B * T, HQ, D, device=device, generator=gen).to(w.dtype)
    sl = torch.full((B,), T, dtype=torch.int32, device=device)
    cu = (torch.arange(B + 1, device=device) * T).to(torch.int32)
    out = torch.empty_like(q)
    flag = torch.zeros(1, dtype=torch.int32, device=device)

    def attn():
        rq.fused_paged_rq_int8_prefill(q, cache, bt, sl, kc, vc, R, H, D, bs, out=out, cu_seqlens_q=cu,
                                       max_q_len=T, error_flag=flag, max_seq_len=T,
                                       staged=not args.fused_prefill)

    def step():
        rq.compress_and_store(key, value, cache, slots, R, kb, vb)
        attn()

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local) if rank == 0 else None
    if world > 1:
        torch.distributed.barrier()
    if sampler:
        sampler.start()
    ms = timed(step, args.steps, device) / args.steps
    attn_ms = timed(attn, args.steps, device) / args.steps
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms, attn_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms, attn_ms = t.tolist()
    if int(flag.item()) != 0:
        raise SystemExit("bench.py: a bounded device-side wait expired in the prefill kernel")
    if rank == 0:
        bf16, kind = 1649.1, "fallback"
        try:
            with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
                bf16, kind = float(json.load(f)["bf16_tflops"]), "measured"
        except (OSError, KeyError, ValueError):
            pass
        peak = 2.0 * bf16           # INT8 dense peak is not measured on this pool: 2 x the bf16 burst figure
        achieved = ops / (attn_ms * 1e-3) / 1e12
        print(json.dumps({
            "metric": "int8_prefill_tokens_per_s", "value": world * B * T / (ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8/bf16",
            "data": "synthetic", "config": workload_config(w, world, B, step=PREFILL_STEP), "clocks": clocks,
            "gpu_launches": (2 if args.fused_prefill else 3) * args.steps,
            "roofline": {"bound": "tensor",
                         "kernel": "prefill_int8_kernel" if args.fused_prefill
                         else "prefill_stage_kernel + prefill_attn_kernel", "achieved": achieved,
                         "peak": peak, "peak_kind": f"2 x {kind} bf16 burst (INT8 peak assumed)",
                         "unit": "TOP/s", "frac": achieved / peak, "kernel_ms": attn_ms,
                         "algorithmic_ops": ops, "traffic": None},
        }))
    if world > 1:
        torch.distributed.destroy_process_group()


def main():
    args = parse_args()
    w = syn.WORKLOADS[args.workload]
    if args.batch > 0:
        import dataclasses

        w = dataclasses.replace(w, batch=args.batch)
    if args.workload == "prefill_int8":
        run_prefill_arm(args, w)
        return
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
