"""Benchmark of the RotorQuant KV-cache hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one attention-layer decode call of the serving path on one batch: compress-on-write
of the step's new K/V tokens into the paged cache, then fused paged decode attention over the
whole compressed context (query rotation, split-KV merge and output rotation included).

* default arm: the CUDA library through its C ABI, one process per GPU (torchrun for N > 1).
  ``value`` is device-resident throughput (inputs already in HBM, CUDA-graph replay), ``e2e`` the
  same step driven from one pinned HOST staging buffer with the host<->device copies inside the
  timed region.  After the timed regions the line also carries, outside any timed region of the
  headline: a parity check of sampled output rows against the CPU oracle, the compress kernel at
  16384 tokens, the INT8 prefill configuration with a measured tensor-pipe peak, the reference's
  own Triton kernels timed on the same inputs, and the head-sharded long-context configuration.
* ``--impl reference``: the reference's CPU path (PyTorch ops, restated in ``oracle/``) on the
  host cores, on a bounded sample of the same workload.

Prints ONE JSON line on rank 0.
"""

from __future__ import annotations

import argparse
import ctypes
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
# DRAM bytes per launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum of the
# attention kernel on the 32-sequence case) divided by the algorithmic bytes of the same launch;
# traffic grows in proportion to the tokens streamed, so the ratio scales `roofline.traffic`.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 158.9e6 / 143.2e6
COMPRESS_BYTES_PER_TOKEN = 5184          # 8 heads x 128 x 2 B x (K, V) read + 1088 B payload written
MIN_TIMED_SECONDS = 0.5


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
    ap.add_argument("--shard-of", type=int, default=0,
                    help="profiling aid for head-sharded workloads on ONE GPU: time the shard rank 0 would hold "
                         "at this world size (no exchange, no extras; the line says so in config.sharding)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--gather", default="both", choices=["both", "peer", "nccl"],
                    help="head-sharded step: exchange head outputs by peer stores, by NCCL all-gather, or time both")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip everything after the headline measurement (profiling runs)")
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


def measured_peaks() -> dict:
    """The pool's measured peaks (HBM copy GB/s, cuBLAS bf16 TFLOP/s), else the stated fallbacks."""
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "kind": "measured"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


def decode_algorithmic_bytes(seq_lens, num_kv_heads: int, num_q_heads: int, block_size: int) -> int:
    """KV payload read once per KV head (136 B per token and head), block-table entries, Q in, O out."""
    total = 0
    for n in seq_lens:
        total += n * num_kv_heads * 136 + ((n + block_size - 1) // block_size) * 4
    total += 2 * len(seq_lens) * num_q_heads * 128 * 2
    return total


def host_threads() -> int:
    """Cores this process may run on.  torchrun exports OMP_NUM_THREADS=1; the CPU arm must use the
    same thread count at every N, so it is set from the affinity mask instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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
        from oracle import rq_oracle  # the CPU arm: the oracle port of the reference's CPU path

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
    torch.set_num_threads(host_threads())
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
    torch.set_num_threads(host_threads())
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
        "config": workload_config(w, max(1, args.gpus), w.batch), "cpu_baseline": base,
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
    """This rank's share of the workload, resident in HBM, plus the step that runs on it.

    ``sharding`` "by sequence": every rank holds its own ``w.batch`` sequences with all heads.
    "by KV head": every rank holds every sequence with ``H / world`` KV heads and their query
    heads (the layout tensor parallelism hands the layer); the head outputs are all-gathered.
    """

    def __init__(self, w: syn.Workload, rank: int, world: int, device: torch.device, sharding: str | None = None,
                 gather_impl: str = "nccl"):
        from rotorquant_vllm import cuda as rq

        self.rq, self.w, self.dev, self.world = rq, w, device, world
        kq, vq, R = make_quantizers(w)
        self.R = R.to(device)
        self.kc, self.vc = kq.centroids.to(device), vq.centroids.to(device)
        self.kb, self.vb = kq.boundaries.to(device), vq.boundaries.to(device)
        self.sharding = sharding or ("by KV head" if w.name == "decode_70b_long" else "by sequence")

        if self.sharding == "by KV head":
            # one request spans the GPUs: every rank sees every sequence
            if w.num_kv_heads % world:
                raise SystemExit(f"{w.name}: {w.num_kv_heads} KV heads do not split over {world} GPUs")
            self.H = w.num_kv_heads // world
            self.HQ = w.num_q_heads // world
            seed = 0
        else:
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

        # ---- per-step inputs: ONE device staging buffer, filled by one host copy in the e2e run ----
        # [q | new K | new V | new slots (int64) | seq_lens (int32) | block-table delta: flat index, value]
        esz = torch.empty(0, dtype=w.dtype).element_size()
        sizes = [B * self.HQ * w.head_dim * esz, B * self.H * w.head_dim * esz, B * self.H * w.head_dim * esz,
                 B * 8, B * 4, B * 8, B * 4]
        offs, total = [], 0
        for n in sizes:
            offs.append(total)
            total += (n + 255) // 256 * 256
        self.staging = torch.zeros(total, dtype=torch.uint8, device=device)

        def view(i, dtype, shape):
            return self.staging[offs[i]:offs[i] + sizes[i]].view(dtype).view(shape)

        self.q = view(0, w.dtype, (B, self.HQ, w.head_dim))
        self.new_k = view(1, w.dtype, (B, self.H, w.head_dim))
        self.new_v = view(2, w.dtype, (B, self.H, w.head_dim))
        self.new_slots = view(3, torch.int64, (B,))
        self.seq_lens = view(4, torch.int32, (B,))
        self.bt_delta_idx = view(5, torch.int64, (B,))       # flat positions in the block table ...
        self.bt_delta_val = view(6, torch.int32, (B,))       # ... and the block numbers to put there

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
            # the table entry a growing sequence would have received this step: its last one
            self.bt_delta_idx[s] = s * self.bt.shape[1] + nb - 1
            self.bt_delta_val[s] = self.bt[s, nb - 1]
        self.q.copy_(torch.randn(B, self.HQ, w.head_dim, device=device, generator=gen).to(w.dtype))
        self.seq_lens.copy_(self.seq_lens_host.to(device))
        self.max_seq_len = int(self.seq_lens_host.max())
        self.gather = None
        self.peer = None                # merge kernel stores into every GPU's buffer + arrive-and-wait kernel
        self.gather_note = None
        if self.sharding == "by KV head" and gather_impl == "peer" and world > 1:
            try:
                self.peer = parallel.PeerHeadGather(B, self.HQ, w.head_dim, w.dtype, device)
            except Exception as exc:    # symmetric memory unavailable on this box: the NCCL form still works
                self.gather_note = f"peer stores unavailable ({type(exc).__name__}: {exc}); NCCL all-gather used"
                print(f"[bench] {self.gather_note}", file=sys.stderr)
        if self.peer is not None:
            self.out = self.peer.begin(0).local
        elif self.sharding == "by KV head":
            self.gather = parallel.HeadGather(B, self.HQ, w.head_dim, w.dtype, device)
            self.out = self.gather.local
        else:
            self.out = torch.empty_like(self.q)
        need_ws = rq.decode_workspace_bytes(B, self.HQ, self.H, w.head_dim, self.max_seq_len)
        self.workspace = torch.empty(max(need_ws, 1), dtype=torch.uint8, device=device)
        torch.cuda.synchronize(device)

    launches_per_step = 3          # compress+store, attention, merge

    def compress(self):
        self.rq.compress_and_store(self.new_k, self.new_v, self.cache, self.new_slots, self.R, self.kb, self.vb)

    def decode_only(self, peer_step=None):
        w = self.w
        if self.peer is not None and peer_step is None:
            peer_step = self.peer.begin(0)
        self.rq.fused_paged_rq_decode(self.q, self.cache, self.bt, self.seq_lens, self.kc, self.vc,
                                      self.R, self.H, w.head_dim, w.block_size,
                                      out=self.out if peer_step is None else peer_step.local,
                                      max_seq_len=self.max_seq_len, workspace=self.workspace,
                                      peer_out_ptrs=None if peer_step is None else peer_step.peer_ptrs)

    def step(self):
        """Device-resident step: compress-on-write, decode, and the exchange of head outputs when sharded by
        head: either the merge kernel's peer stores + one arrive-and-wait kernel (two gathered buffers
        alternate from step to step), or one in-place NCCL all-gather."""
        self.compress()
        if self.peer is not None:
            self.decode_only(self.peer.begin())
            self.peer.finish()
            return
        self.decode_only()
        if self.gather is not None:
            self.gather.gather()

    @property
    def gathered(self):
        """The buffer an end-to-end step reads back."""
        if self.peer is not None:
            return self.peer.buffer[0]
        return self.gather.buffer if self.gather is not None else self.out

    def step_with_table_update(self):
        """The step as the serving loop runs it: the block-table entries that changed are applied first."""
        self.bt.view(-1).index_copy_(0, self.bt_delta_idx, self.bt_delta_val)
        self.step()

    def algorithmic_bytes(self) -> int:
        return decode_algorithmic_bytes(self.seq_lens_host.tolist(), self.H, self.HQ, self.w.block_size)

    def parity_check(self, sample_seqs: int = 2) -> dict:
        """Compare the output rows of a few sequences with the CPU oracle (outside any timed region)."""
        from oracle import rq_oracle, tolerance  # checker only

        w, bs = self.w, self.w.block_size
        self.decode_only()
        torch.cuda.synchronize(self.dev)
        out = self.out.cpu()
        kc, vc, R = self.kc.cpu(), self.vc.cpu(), self.R.cpu()
        n_seqs = len(self.seq_lens_host)
        k = max(1, min(sample_seqs, n_seqs))
        picks = sorted({round(i * (n_seqs - 1) / max(k - 1, 1)) for i in range(k)})   # evenly spread, ends included
        worst, over, rows = 0.0, 0, 0
        for s in picks:
            n = int(self.seq_lens_host[s])
            nb = (n + bs - 1) // bs
            sub = self.cache[self.bt[s, :nb].long()].cpu()
            table = torch.arange(nb, dtype=torch.int32).unsqueeze(0)
            lens = torch.tensor([n], dtype=torch.int32)
            q = self.q[s:s + 1].cpu()
            ref = rq_oracle.decode(q, sub, table, lens, kc, vc, R, self.H, w.head_dim, bs)
            rot = rq_oracle.decode(q, sub, table, lens, kc, vc, R, self.H, w.head_dim, bs, return_rotated_fp32=True)
            m, bad = tolerance.excess(out[s:s + 1], rot, ref, w.dtype)
            worst, over, rows = max(worst, m), over + bad, rows + self.HQ
        return {"rows": rows, "sequences": picks, "max_abs": worst, "over_tolerance": over,
                "against": "oracle/rq_oracle.decode (reference decompress + SDPA), bound 2e-3 or one rounding flip"}


def timed(fn, steps: int, device, tail=None) -> float:
    """Milliseconds for `steps` calls of fn, CUDA events on the current stream.  `tail`, when given, runs
    after the last call and before the closing event (it makes the current stream wait for work that fn
    put on another stream, so that the event covers it)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(device)
    e0.record()
    for _ in range(steps):
        fn()
    if tail is not None:
        tail()
    e1.record()
    torch.cuda.synchronize(device)
    return e0.elapsed_time(e1)


def timed_chunks(fn, steps: int, device, min_seconds: float = MIN_TIMED_SECONDS, max_chunks: int = 400, tail=None,
                 agree=None):
    """Time chunks of exactly `steps` calls until at least `min_seconds` have been measured;
    returns (median chunk in ms, number of chunks).  `agree(n) -> n` makes the ranks of a job settle on
    one chunk count: every rank must run a step that holds an exchange the same number of times."""
    first = timed(fn, steps, device, tail)
    chunks = [first]
    want = min(max_chunks, max(1, math.ceil(min_seconds * 1e3 / max(first, 1e-3))))
    if agree is not None:
        want = agree(want)
    while len(chunks) < want:
        chunks.append(timed(fn, steps, device, tail))
    return statistics.median(chunks), len(chunks)


def capture(fn, device, what: str):
    """CUDA graph of one call of fn, or None when capture is unavailable."""
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize(device)
        return graph
    except Exception as exc:  # capture is an optimisation of the launch path only
        print(f"[bench] CUDA graph capture of {what} unavailable ({exc}); launching directly", file=sys.stderr)
        torch.cuda.synchronize(device)
        return None


def measure_job(job: GpuJob, args, device, barrier, world: int, sampler=None) -> dict:
    """Device-resident throughput, decode-kernel time and end-to-end time of one job (all max over ranks
    is taken by the caller)."""
    dist = torch.distributed
    for _ in range(max(args.warmup, 3)):
        job.step()
    graph = None if args.no_graph else capture(job.step, device, "the step")
    runner = graph.replay if graph is not None else job.step
    if graph is not None and job.peer is not None:
        # the peer-store form alternates two gathered buffers: one graph per parity, replayed in turn
        graph2 = capture(job.step, device, "the step (second gathered buffer)")
        if graph2 is not None:
            pair, turn_g = (graph, graph2), [0]

            def runner():
                pair[turn_g[0]].replay()
                turn_g[0] ^= 1
    barrier()
    if sampler:
        sampler.start()
    def agree(n: int) -> int:                   # the largest count any rank wants
        if world == 1:
            return n
        t = torch.tensor([n], dtype=torch.int64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return int(t.item())

    ms_chunk, n_chunks = timed_chunks(runner, args.steps, device, agree=agree)
    barrier()

    # ---- the dominant kernel alone (attention + merge), same inputs: in a graph, and launched one by one ----
    job.compress()
    dgraph = None if args.no_graph else capture(job.decode_only, device, "the decode launches")
    decode_graph_ms = None
    if dgraph is not None:
        decode_graph_ms = timed_chunks(dgraph.replay, args.steps, device, 0.2, agree=agree)[0] / args.steps
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(min(args.steps, 200))]
    torch.cuda.synchronize(device)
    for a, b in evs:
        job.compress()
        a.record()
        job.decode_only()
        b.record()
    torch.cuda.synchronize(device)
    decode_eager_ms = statistics.mean(a.elapsed_time(b) for a, b in evs)
    compress_ms = timed(job.compress, min(args.steps, 200), device) / min(args.steps, 200)
    # the step without its collective, to price the gather
    nogather_ms = None
    if (job.gather is not None or job.peer is not None) and world > 1:
        g2 = None if args.no_graph else capture(lambda: (job.compress(), job.decode_only()), device, "the step without gather")
        fn = g2.replay if g2 is not None else (lambda: (job.compress(), job.decode_only()))
        nogather_ms = timed_chunks(fn, args.steps, device, 0.2, agree=agree)[0] / args.steps
    clocks = sampler.stop() if sampler else None

    # ---- end to end: ONE pinned host buffer -> device staging, table update + step, ONE read back ----
    host_in = job.staging.cpu().pin_memory()
    result = job.gathered
    host_out = torch.empty(result.shape, dtype=result.dtype).pin_memory()
    egraph = None if args.no_graph else capture(job.step_with_table_update, device, "the end-to-end step")
    erun = egraph.replay if egraph is not None else job.step_with_table_update

    # Serial form first (one stream: upload, step, read-back), reported beside the pipelined number.
    def e2e_serial_step():
        job.staging.copy_(host_in, non_blocking=True)
        erun()
        host_out.copy_(result, non_blocking=True)

    for _ in range(3):
        e2e_serial_step()
    e2e_serial_ms = timed_chunks(e2e_serial_step, args.steps, device, 0.2, agree=agree)[0]

    # Pipelined form: PCIe is full duplex and the copy engines run beside the SMs, so the inputs of step
    # i + 1 are uploaded (into one of two landing buffers, on an upload stream) and the output of step i - 1
    # is read back (on a read-back stream) while step i computes.  On the compute stream a step is: copy the
    # landing buffer into the staging buffer the graph reads, wait until the previous read-back has finished
    # with the output buffer, replay the graph.  Every step's inputs still cross PCIe from pinned host
    # memory and every step's output still reaches the host inside the timed region.
    main = torch.cuda.current_stream(device)
    uploader, reader = torch.cuda.Stream(device), torch.cuda.Stream(device)
    landing = [job.staging.clone() for _ in range(2)]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    computed, read_back = torch.cuda.Event(), torch.cuda.Event()
    read_back.record(main)
    for ev in consumed:
        ev.record(main)
    turn = [0]

    def e2e_step():
        b = turn[0]
        turn[0] ^= 1
        uploader.wait_event(consumed[b])
        with torch.cuda.stream(uploader):
            landing[b].copy_(host_in, non_blocking=True)
            uploaded[b].record(uploader)
        main.wait_event(uploaded[b])
        job.staging.copy_(landing[b], non_blocking=True)
        consumed[b].record(main)
        main.wait_event(read_back)
        erun()
        computed.record(main)
        reader.wait_event(computed)
        with torch.cuda.stream(reader):
            host_out.copy_(result, non_blocking=True)
            read_back.record(reader)

    def e2e_tail():
        main.wait_event(read_back)            # the closing event covers the last read-back

    # Jobs without an exchange get a leaner pipeline, because the form above is bound by the dozen stream
    # operations Python issues per step: two graphs (one per landing buffer and output buffer) that begin
    # with the copy of their landing buffer into the staging buffer, and ONE copy stream that, after step i,
    # reads its output back and uploads the inputs of step i + 2 into the landing buffer step i has consumed.
    # Seven stream operations per step; every step still has its own upload and its own read-back in the region.
    if egraph is not None and job.gather is None and job.peer is None:
        # the landing buffers hold real inputs before anything replays a graph that reads them
        for b in range(2):
            landing[b].copy_(host_in, non_blocking=True)
        torch.cuda.synchronize(device)
        outs = [job.out, torch.empty_like(job.out)]
        pair = []
        for b in range(2):
            job.out = outs[b]

            def step_b(b=b):
                job.staging.copy_(landing[b], non_blocking=True)
                job.step_with_table_update()

            pair.append(capture(step_b, device, f"the end-to-end step ({b})"))
        job.out = outs[0]
        if all(g is not None for g in pair):
            landed = [torch.cuda.Event() for _ in range(2)]
            finished = [torch.cuda.Event() for _ in range(2)]
            with torch.cuda.stream(uploader):
                for b in range(2):
                    landing[b].copy_(host_in, non_blocking=True)
                    landed[b].record(uploader)
            torch.cuda.synchronize(device)
            turn[0] = 0

            def e2e_step():                               # noqa: F811  (replaces the general form)
                b = turn[0]
                turn[0] ^= 1
                main.wait_event(landed[b])
                pair[b].replay()
                finished[b].record(main)
                uploader.wait_event(finished[b])
                with torch.cuda.stream(uploader):
                    host_out.copy_(outs[b], non_blocking=True)
                    landing[b].copy_(host_in, non_blocking=True)
                    landed[b].record(uploader)

            def e2e_tail():                               # noqa: F811
                main.wait_event(landed[0])
                main.wait_event(landed[1])

    for _ in range(4):
        e2e_step()
    barrier()
    e2e_ms = timed_chunks(e2e_step, args.steps, device, tail=e2e_tail, agree=agree)[0]
    barrier()
    e2e_tail()
    torch.cuda.synchronize(device)
    # what reached the host is what the device holds (outside the timed region)
    read_back_ok = bool(torch.equal(host_out, result.cpu()))

    t = torch.tensor([ms_chunk, e2e_ms, decode_eager_ms, decode_graph_ms or decode_eager_ms, compress_ms,
                      nogather_ms or 0.0, e2e_serial_ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_chunk, e2e_ms, decode_eager_ms, decode_kernel_ms, compress_ms, nogather_ms, e2e_serial_ms = t.tolist()
    return {"ms_per_step": ms_chunk / args.steps, "chunks": n_chunks, "e2e_ms_per_step": e2e_ms / args.steps,
            "e2e_serial_ms_per_step": e2e_serial_ms / args.steps,
            "decode_kernel_ms": decode_kernel_ms, "decode_kernel_ms_eager": decode_eager_ms,
            "decode_in_graph": dgraph is not None, "compress_ms": compress_ms,
            "nogather_ms": nogather_ms if nogather_ms > 0 else None, "clocks": clocks,
            "graph": graph is not None, "h2d": host_in.numel(), "d2h": host_out.numel() * host_out.element_size(),
            "read_back_ok": read_back_ok}


# --------------------------------------------------------------------------------------------
# Secondary measurements (after the headline, outside its timed regions)
# --------------------------------------------------------------------------------------------

def measure_tensor_peaks(device) -> dict:
    """Tensor-pipe rates of this GPU from the library's probe: back-to-back tcgen05 MMAs of one kind."""
    from rotorquant_vllm import _lib

    lib = _lib.lib()
    flag = torch.zeros(1, dtype=torch.int32, device=device)
    out = {}
    for kind, name in ((0, "int8_tops"), (1, "bf16_tflops_mma")):
        ops = ctypes.c_double(0.0)
        stream = torch.cuda.current_stream(device).cuda_stream

        def run(iters):
            _lib.check(lib.rq_probe_mma_peak(kind, iters, ctypes.byref(ops), flag.data_ptr(), stream))

        run(256)
        torch.cuda.synchronize(device)
        best = 0.0
        for _ in range(5):
            ms = timed(lambda: run(4096), 1, device)
            best = max(best, ops.value / (ms * 1e-3) / 1e12)
        out[name] = best
    out["probe_wait_expired"] = bool(int(flag.item()))
    out["how"] = ("rq_probe_mma_peak: one CTA per SM issues 16384 back-to-back 128x256x32-byte tcgen05.mma "
                  "from shared memory into two TMEM accumulators, best of 5, CUDA events")
    return out


def measure_compress(job: GpuJob, device, tokens: int = 16384) -> dict:
    """compress_store on `tokens` new tokens (8 KV heads): the BASELINE metric's "compress Mtok/s"."""
    w = job.w
    gen = torch.Generator(device=device).manual_seed(4242)
    k = torch.randn(tokens, job.H, w.head_dim, device=device, generator=gen)
    v = torch.randn(tokens, job.H, w.head_dim, device=device, generator=gen)
    k[..., 3] *= 10
    v[..., 3] *= 10
    k, v = k.to(w.dtype), v.to(w.dtype)
    nslots = job.cache.shape[0] * job.cache.shape[1]
    slots = torch.randperm(nslots, device=device, generator=gen)[:tokens].to(torch.int64)
    saved = job.cache.view(-1, job.cache.shape[2])[slots].clone()

    def run():
        job.rq.compress_and_store(k, v, job.cache, slots, job.R, job.kb, job.vb)

    for _ in range(3):
        run()
    ms = timed_chunks(run, 20, device, 0.1)[0] / 20
    job.cache.view(-1, job.cache.shape[2])[slots] = saved
    peak = measured_peaks()
    bytes_per_token = job.H * (2 * w.head_dim * 2 + 136)
    gbs = tokens * bytes_per_token / (ms * 1e-3) / 1e9
    return {"tokens": tokens, "kv_heads": job.H, "ms": ms, "mtok_per_s": tokens / (ms * 1e-3) / 1e6,
            "roofline": {"bound": "hbm", "kernel": "compress_store_kernel", "achieved": gbs, "peak": peak["hbm_gbs"],
                         "unit": "GB/s", "frac": gbs / peak["hbm_gbs"], "peak_kind": peak["kind"] + " copy bandwidth",
                         "algorithmic_bytes_per_token": bytes_per_token},
            "_inputs": (k, v, slots)}


class PrefillJob:
    """The INT8 prefill configuration: B causal sequences of T new tokens, compress-on-write + attention."""

    def __init__(self, w: syn.Workload, rank: int, device):
        from rotorquant_vllm import cuda as rq

        self.rq, self.w, self.dev = rq, w, device
        T, B, H, HQ, D, bs = w.ctx_max, w.batch, w.num_kv_heads, w.num_q_heads, w.head_dim, w.block_size
        kq, vq, R = make_quantizers(w)
        self.R = R.to(device)
        self.kc, self.vc, self.kb, self.vb = (t.to(device) for t in (kq.centroids, vq.centroids, kq.boundaries, vq.boundaries))
        gen = torch.Generator(device=device).manual_seed(rank)
        nblk = B * T // bs
        self.cache = torch.zeros(nblk, bs, H * 256, dtype=torch.uint8, device=device)
        self.bt = torch.randperm(nblk, device=device, generator=gen).to(torch.int32).reshape(B, T // bs).contiguous()
        pos = torch.arange(T, device=device)
        self.slots = torch.cat([self.bt[s].long()[pos // bs] * bs + pos % bs for s in range(B)])
        key = torch.randn(B * T, H, D, device=device, generator=gen)
        value = torch.randn(B * T, H, D, device=device, generator=gen)
        key[..., 3] *= 10
        value[..., 3] *= 10
        self.key, self.value = key.to(w.dtype), value.to(w.dtype)
        self.q = torch.randn(B * T, HQ, D, device=device, generator=gen).to(w.dtype)
        self.sl = torch.full((B,), T, dtype=torch.int32, device=device)
        self.cu = (torch.arange(B + 1, device=device) * T).to(torch.int32)
        self.out = torch.empty_like(self.q)
        self.flag = torch.zeros(1, dtype=torch.int32, device=device)
        self.ops = 4 * D * B * HQ * T * (T + 1) // 2          # causal, QK^T + PV, 2 per multiply-add

    def attn(self, staged=True):
        w = self.w
        self.rq.fused_paged_rq_int8_prefill(self.q, self.cache, self.bt, self.sl, self.kc, self.vc, self.R,
                                            w.num_kv_heads, w.head_dim, w.block_size, out=self.out,
                                            cu_seqlens_q=self.cu, max_q_len=w.ctx_max, error_flag=self.flag,
                                            max_seq_len=w.ctx_max, staged=staged)

    def compress(self):
        self.rq.compress_and_store(self.key, self.value, self.cache, self.slots, self.R, self.kb, self.vb)

    def step(self, staged=True):
        self.compress()
        self.attn(staged)


def prefill_roofline(ops: int, attn_ms: float, peaks: dict) -> dict:
    """Achieved tensor rate of the prefill attention against the measured pipe rates: half of the
    operations (Q K^T) run on the INT8 path, half (P V) on the 16-bit path, so the roof of the mix is
    2 / (1 / int8 + 1 / bf16)."""
    achieved = ops / (attn_ms * 1e-3) / 1e12
    int8, bf16 = peaks["int8_tops"], peaks["bf16_tflops_mma"]
    mixed = 2.0 / (1.0 / int8 + 1.0 / bf16)
    return {"bound": "tensor", "kernel": "prefill_stage_kernel + prefill_attn_kernel", "achieved": achieved,
            "peak": mixed, "unit": "TOP/s", "frac": achieved / mixed, "frac_of_int8_peak": achieved / int8,
            "int8_tops": int8, "bf16_tflops_mma": bf16,
            "peak_kind": "measured tcgen05 pipe rates (rq_probe_mma_peak), mixed INT8 / bf16 roof",
            "kernel_ms": attn_ms, "algorithmic_ops": ops, "traffic": None}


def measure_prefill(device, peaks: dict, steps: int = 10) -> dict:
    w = syn.WORKLOADS["prefill_int8"]
    job = PrefillJob(w, 0, device)
    for _ in range(3):
        job.step()
    ms = timed_chunks(job.step, steps, device, 0.1)[0] / steps
    attn_ms = timed_chunks(job.attn, steps, device, 0.1)[0] / steps
    if int(job.flag.item()) != 0:
        return {"error": "a bounded device-side wait expired in the prefill kernel"}
    return {"workload": "prefill_int8: 8 causal sequences x 2048 new tokens, 32 query / 8 KV heads, iso-fast 3-bit",
            "tokens_per_s": w.batch * w.ctx_max / (ms * 1e-3), "ms_per_step": ms,
            "step": PREFILL_STEP, "roofline": prefill_roofline(job.ops, attn_ms, peaks), "_job": job}


def measure_triton_baseline(job: GpuJob, compress_inputs, prefill_job, device, steps: int) -> dict:
    """The reference's own Triton kernels (compiled for this GPU by Triton's JIT) timed with the same
    events on the same inputs as the new kernels: the existing-GPU-kernel bar."""
    sys.path.insert(0, REPO)
    try:
        from baseline import ref_kernels
    except Exception as exc:
        return {"unavailable": f"baseline/ref_kernels.py not importable: {exc}"}
    if not ref_kernels.available():
        return {"unavailable": "baseline/_ref is not installed (see baseline/ref_kernels.py)"}
    out: dict = {"source": "unmodified reference package under baseline/_ref, Triton JIT for this GPU"}
    w = job.w
    # decode: the reference launcher (two dense rotations + one kernel) on this job's cache and queries
    try:
        ref_decode = ref_kernels.load("fused_paged_rq_decode")
        ref_out = torch.empty_like(job.q)

        def dec():
            ref_decode(job.q, job.cache, job.bt, job.seq_lens, job.kc, job.vc, job.R, job.H, w.head_dim,
                       w.block_size, out=ref_out)

        for _ in range(3):
            dec()
        n = max(3, min(steps, 20))
        ms = timed(dec, n, device) / n
        job.decode_only()
        torch.cuda.synchronize(device)
        diff = (ref_out.float() - job.out.float()).abs().max().item()
        out["decode"] = {"ms": ms, "tokens_per_s": w.batch / (ms * 1e-3),
                         "gbs": job.algorithmic_bytes() / (ms * 1e-3) / 1e9, "max_abs_vs_new_kernel": diff}
    except Exception as exc:
        out["decode"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    # compress: iso_compress on K and on V (the reference then assembles rows and scatters in PyTorch)
    try:
        k, v, _slots = compress_inputs
        ref_compress = ref_kernels.load("iso_compress" if w.rq_mode == "iso" else "planar_compress")
        rot_t = job.R.T.contiguous()
        even, odd = rot_t[:, 0::2].contiguous(), rot_t[:, 1::2].contiguous()

        def comp():
            ref_compress(k, even, odd, job.kb)
            ref_compress(v, even, odd, job.vb)

        for _ in range(3):
            comp()
        ms = timed(comp, 20, device) / 20
        out["compress"] = {"tokens": k.shape[0], "ms": ms, "mtok_per_s": k.shape[0] / (ms * 1e-3) / 1e6,
                           "note": "two kernel launches only; the reference's row assembly and scatter are not included"}
    except Exception as exc:
        out["compress"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    # prefill: the reference kernel is single-sequence, so one call per sequence as its backend does
    try:
        pj = prefill_job
        if pj is None:
            raise RuntimeError("prefill job not built")
        ref_prefill = ref_kernels.load("fused_paged_rq_int8_prefill")
        T, B = pj.w.ctx_max, pj.w.batch
        ref_o = torch.empty_like(pj.q)

        def pre():
            for s in range(B):
                ref_prefill(pj.q[s * T:(s + 1) * T], pj.cache, pj.bt[s:s + 1], pj.sl[s:s + 1], pj.kc, pj.vc,
                            pj.R, pj.w.num_kv_heads, pj.w.head_dim, pj.w.block_size, out=ref_o[s * T:(s + 1) * T])

        pre()
        pre()
        ms = timed(pre, 3, device) / 3
        out["prefill"] = {"ms": ms, "tokens_per_s": B * T / (ms * 1e-3), "tops": pj.ops / (ms * 1e-3) / 1e12,
                          "note": "attention only (no compress), 8 launches of the single-sequence kernel"}
    except Exception as exc:
        out["prefill"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}
    return out


def measure_strong(args, rank: int, world: int, device, barrier) -> dict:
    """The long-context configuration sharded by KV head with its one all-gather (strong scaling): at
    N GPUs every rank holds 8 / N KV heads of all 8 sequences of 131072 tokens."""
    w = syn.WORKLOADS["decode_70b_long"]
    if w.num_kv_heads % world:
        return {"unavailable": f"{w.num_kv_heads} KV heads do not split over {world} GPUs"}
    dist = torch.distributed
    sub = argparse.Namespace(**vars(args))
    sub.steps = max(10, min(args.steps, 100))
    peak = measured_peaks()
    forms = ["peer", "nccl"] if world > 1 else ["nccl"]
    if getattr(args, "gather", "both") in ("peer", "nccl") and world > 1:
        forms = [args.gather]
    out = {}
    for form in forms:
        job = GpuJob(w, rank, world, device, sharding="by KV head", gather_impl=form)
        if form == "peer" and job.peer is None:
            out["peer"] = {"unavailable": job.gather_note}
            del job
            torch.cuda.empty_cache()
            continue
        m = measure_job(job, sub, device, barrier, world)
        alg = job.algorithmic_bytes()
        gbs = alg / (m["decode_kernel_ms"] * 1e-3) / 1e9
        how = ("merge kernel stores every output row into all GPUs' gathered buffers (peer memory over NVLink) + "
               "one arrive-and-wait kernel" if form == "peer" else "one in-place NCCL all-gather of head outputs")
        res = {"workload": w.name, "sharding": "by KV head; " + how,
               "kv_heads_per_gpu": job.H, "q_heads_per_gpu": job.HQ, "num_seqs": w.batch, "context": w.ctx_max,
               "kernel_us": m["decode_kernel_ms"] * 1e3, "step_us": m["ms_per_step"] * 1e3,
               "gather_us": (m["ms_per_step"] - m["nogather_ms"]) * 1e3 if m["nogather_ms"] else 0.0,
               "e2e_step_us": m["e2e_ms_per_step"] * 1e3, "tokens_per_s": w.batch / (m["ms_per_step"] * 1e-3),
               "algorithmic_bytes_per_gpu": alg, "achieved_gbs": gbs, "frac": gbs / peak["hbm_gbs"],
               "cuda_graph": m["graph"]}
        if world > 1:
            # the gathered buffer of one more step against an NCCL all-gather of the local head outputs
            barrier()
            if job.peer is not None:
                par = job.peer.parity
                job.step()
                torch.cuda.synchronize(device)
                got, local = job.peer.buffer[par], job.peer.buffer[par, rank]
            else:
                job.step()
                torch.cuda.synchronize(device)
                got, local = job.gather.buffer, job.gather.local
            ref = torch.empty_like(got)
            dist.all_gather_into_tensor(ref.view(-1, *local.shape[1:]), local.contiguous())
            ok = torch.tensor([1 if torch.equal(got, ref) else 0], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            res["gathered_equals_all_gather_on_every_rank"] = bool(ok.item())
            if job.peer is not None:
                bad = torch.tensor([1 if job.peer.wait_expired() else 0], device=device)
                dist.all_reduce(bad, op=dist.ReduceOp.MAX)
                res["a_bounded_wait_expired"] = bool(bad.item())
        if rank == 0:
            res["parity_check"] = job.parity_check(1)
        out[form] = res
        del job
        torch.cuda.empty_cache()
        barrier()
    head = out.get("peer") if "step_us" in out.get("peer", {}) else out.get("nccl")
    res = dict(head) if head else {"unavailable": "no form of the head-sharded step ran"}
    if "nccl" in out and head is not out.get("nccl"):
        res["nccl_all_gather_form"] = {k: out["nccl"][k] for k in ("step_us", "gather_us", "kernel_us", "tokens_per_s",
                                                                    "gathered_equals_all_gather_on_every_rank")
                                       if k in out["nccl"]}
    if "peer" in out and "unavailable" in out["peer"]:
        res["peer_store_form"] = out["peer"]
    return res


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

    shard_of = args.shard_of if (world == 1 and args.shard_of > 1) else 0
    job = GpuJob(w, rank, shard_of or world, device, sharding="by KV head" if shard_of else None)
    if shard_of:
        job.gather = None
        job.out = job.out.clone()
        args.no_extras = True
    sampler = ClockSampler(local) if rank == 0 else None
    m = measure_job(job, args, device, barrier, world, sampler)

    line = None
    if rank == 0:
        seqs_per_step = w.batch * (world if job.sharding == "by sequence" else 1)
        peak = measured_peaks()
        alg = job.algorithmic_bytes()
        achieved = alg / (m["decode_kernel_ms"] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": seqs_per_step / (m["ms_per_step"] * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": m["ms_per_step"], "timed_chunks_of_steps": m["chunks"], "higher_is_better": True,
            "scaling": "weak" if job.sharding == "by sequence" else "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": workload_config(w, world, w.batch, job.sharding if not shard_of else
                                      f"the shard of rank 0 of {shard_of} by KV head ({job.H} KV heads), no exchange"),
            "clocks": m["clocks"], "cuda_graph": m["graph"],
            "e2e": {"value": seqs_per_step / (m["e2e_ms_per_step"] * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": m["h2d"], "d2h_bytes_per_step": m["d2h"],
                    "serial_value": seqs_per_step / (m["e2e_serial_ms_per_step"] * 1e-3),
                    "read_back_equals_device_output": m["read_back_ok"],
                    "how": "per step: one pinned staging buffer -> one H2D copy, graph replay (block-table delta + "
                           "compress + decode), one D2H copy of the output; pipelined over steps (copy stream and "
                           "compute stream, two landing buffers and two output buffers), so a step's copies overlap "
                           "its neighbours' compute; serial_value is the same without overlap (one stream)"},
            "gpu_launches": job.launches_per_step * args.steps * m["chunks"],
            "roofline": {"bound": "hbm", "kernel": "decode_attn_kernel (+ merge kernel)",
                         "achieved": achieved, "peak": peak["hbm_gbs"], "peak_kind": f"{peak['kind']} copy bandwidth",
                         "unit": "GB/s", "frac": achieved / peak["hbm_gbs"],
                         "algorithmic_bytes": alg, "kernel_ms": m["decode_kernel_ms"],
                         "kernel_ms_how": "graph replay of the decode launches" if m["decode_in_graph"] else "events around eager launches",
                         "kernel_ms_eager": m["decode_kernel_ms_eager"],
                         "traffic": alg * NCU_TRAFFIC_PER_ALGORITHMIC_BYTE},
            "decode_tokens_per_s_per_gpu": w.batch / (m["decode_kernel_ms"] * 1e-3),
            "compress_mtok_per_s_at_decode_batch": w.batch / (m["compress_ms"] * 1e-3) / 1e6,
        }
    if not args.no_extras:
        if rank == 0:
            line["parity_check"] = job.parity_check()
            comp = measure_compress(job, device) if job.sharding == "by sequence" else None
            if world == 1:
                try:
                    tp = measure_tensor_peaks(device)
                    pf = measure_prefill(device, tp)
                except Exception as exc:
                    tp, pf = None, {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}
                line["tensor_peaks"] = tp
                line["triton_baseline"] = measure_triton_baseline(
                    job, comp["_inputs"] if comp else None, pf.get("_job") if isinstance(pf, dict) else None,
                    device, args.steps)
                pf.pop("_job", None)
                line["prefill"] = pf
            if comp:
                comp.pop("_inputs", None)
                line["compress"] = comp
        # every rank takes part in the head-sharded configuration
        if w.name != "decode_70b_long":
            del job
            torch.cuda.empty_cache()
            barrier()
            strong = measure_strong(args, rank, world, device, barrier)
            if rank == 0:
                line["strong"] = strong
    if rank == 0:
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
    if args.impl == "reference":
        if rank != 0:
            return
        from oracle import rq_oracle

        torch.set_num_threads(host_threads())
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

    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=device)
    job = PrefillJob(w, rank, device)
    staged = not args.fused_prefill

    for _ in range(max(args.warmup, 3)):
        job.step(staged)
    sampler = ClockSampler(local) if rank == 0 else None
    if world > 1:
        torch.distributed.barrier()
    if sampler:
        sampler.start()
    ms = timed_chunks(lambda: job.step(staged), args.steps, device)[0] / args.steps
    attn_ms = timed_chunks(lambda: job.attn(staged), args.steps, device)[0] / args.steps
    clocks = sampler.stop() if sampler else None
    t = torch.tensor([ms, attn_ms], dtype=torch.float64, device=device)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms, attn_ms = t.tolist()
    if int(job.flag.item()) != 0:
        raise SystemExit("bench.py: a bounded device-side wait expired in the prefill kernel")
    if rank == 0:
        roof = prefill_roofline(job.ops, attn_ms, measure_tensor_peaks(device))
        if args.fused_prefill:
            roof["kernel"] = "prefill_int8_kernel"
        print(json.dumps({
            "metric": "int8_prefill_tokens_per_s", "value": world * B * T / (ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "s8/bf16",
            "data": "synthetic", "config": workload_config(w, world, B, step=PREFILL_STEP), "clocks": clocks,
            "gpu_launches": (2 if args.fused_prefill else 3) * args.steps,
            "roofline": roof,
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
