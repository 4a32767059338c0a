"""Benchmark of the attention hot path on synthetic inputs of the reference's headline shapes.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Prints ONE JSON line.  Workloads (shapes of the five benchmark configurations):
    prefill_causal  B4 S8192 H8 G2 D256 bf16, causal, scale 1/16          (default, headline)
    prefill_swa     B2 S32768 W512, per-query sliding window
    decode_paged    256 sequences, ctx ~ U[1024,32768], fp16 KV in shuffled 16-token pages,
                    one step = append the new token's K/V + attention
    decode_long     1 sequence of 131072 tokens, bf16 paged KV; with N > 1 the KV range is
                    split across GPUs and the (acc, l, m) partials are merged across them
    prefill_chunk   256 new rows of one request over 65536 cached keys (split-KV over the SMs;
                    --kv-splits -1 runs it unsplit)
    rope_append     the launch before attention: norm + rotary embedding + KV append, GB/s
    kv_append       add_kv_to_cache alone on a prefill chunk (V norm, f32 -> f16), GB/s
    decode_paged_fp8  decode_paged over 8-bit (e4m3) pages with a scale per (page, kv head):
                    1024 bytes of K/V per token instead of 2048
A step is one pass of the hot path over one batch.  ``value`` has inputs resident in HBM;
``e2e`` goes through the public Python operators with pinned host buffers, host<->device
copies inside the timed region.

The default line is the headline (prefill_causal, the same per-GPU batch on every rank: weak
scaling) plus one block per other configuration, each with its own time, roofline and a
parity check against the CPU oracle made in this run:
    swa          configuration 3; on N > 1 GPUs its (request, kv head) units, and at 8 GPUs
                 halves of their query range with a window-sized key halo, are dealt over the
                 ranks (strong scaling, no communication)
    decode       configuration 4; on N > 1 GPUs ONE set of 256 sequences dealt over the ranks
                 longest-first (strong scaling, no communication)
    decode_fp8   configuration 4 over 8-bit (e4m3) pages with a scale per (page, kv head); GB/s of
                 the bytes it reads, half of configuration 4's
    decode_long  configuration 5; on N > 1 GPUs the KV range of the one sequence is split over
                 the ranks and the partials are merged through peer memory (strong scaling, the
                 one exchange step of the path); every rank checks its output against the oracle
    prefill_strong (N > 1 only) configuration 2's ONE batch of 4 requests dealt over the ranks
                 by request and kv head
plus ``sustained`` (the headline replayed for two seconds with the clocks sampled),
``copy_ceiling`` (what the same pinned buffers reach with copies alone), ``cpu_config1`` (the
reference's CPU case, configuration 1, timed in full) and ``triton_reference`` (the
reference's own Triton kernel on the same GPU, when its sources were copied beside the repo).
``--impl reference`` times the reference's CPU attention on the host cores over the whole
per-GPU batch of the workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

H, G, D, PAGE = 8, 2, 256, 16
SCALE = 1.0 / 16.0


# ------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------
def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), tensor=float(d["bf16_tflops"]),
                    tensor_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, tensor=1590.0, tensor_sustained=1400.0, source="fallback")


def captured_traffic(workload: str):
    """DRAM bytes (read + write) that the profiler counted for one launch of the workload's
    dominant kernel, from the record kept beside the profile summaries: {"bytes_per_unit",
    "fixed_bytes", "units"}; traffic of a launch = bytes_per_unit * units + fixed_bytes.  None
    where no capture exists."""
    p = ROOT / "profiles" / "traffic.json"
    if not p.exists():
        return None
    return json.loads(p.read_text()).get(workload)


class ClockSampler:
    """Polls SM clock, power and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.power, self.reasons, self.max_mhz = [], [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:  # NVML missing: report no clocks rather than fail the bench
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()
        s, w = sorted(self.samples), sorted(self.power)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s),
                "power_w": (round(w[len(w) // 2], 1) if w else None)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def barrier_sync(world):
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int, dev) -> float:
    if world == 1:
        return ms
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


def all_ranks_ok(ok: bool, world: int, dev) -> bool:
    if world == 1:
        return ok
    t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MIN)
    return bool(t.item())


def timed_region(step_fn, steps, warmup, world, dev, sampler=None, begin=None, end=None):
    """W warm-up steps, then exactly K steps between CUDA events on the launching stream,
    bracketed by barrier + synchronize; returns the max over ranks in ms."""
    if begin is not None:
        begin()
    many = getattr(step_fn, "run_many", None)
    if many is not None:
        many(0, warmup)
    else:
        for i in range(warmup):
            step_fn(i)
    if end is not None:
        end()
    barrier_sync(world)
    if sampler is not None:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if many is not None:
        many(warmup, steps)
    else:
        for i in range(steps):
            step_fn(warmup + i)
    if end is not None:
        end()                     # side streams join the launching stream before the stop event
    e1.record()
    barrier_sync(world)
    ms = e0.elapsed_time(e1)
    return max_over_ranks(ms, world, dev)


class GraphRunner:
    """Replays a step from CUDA graphs (one per input variant), as the reference engine does
    in deployment (g4b/lifecycle.py:39-51): the operators neither allocate nor synchronise, so
    a step is capturable, and replay removes the Python launch overhead that otherwise
    dominates microsecond-scale decode steps.  A workload that rotates over several input
    variants also gets graphs that hold GROUP consecutive steps (consecutive variants, back to
    back): the engine's graph holds a model step with one attention call per layer, so
    consecutive calls there are graph nodes too, not separate graph launches.  Falls back to
    direct launches if capture fails."""

    GROUP = 4

    def __init__(self, step_fn, variants: int, enabled: bool):
        self.step_fn, self.graphs, self.groups, self.mode = step_fn, [], {}, "direct"
        if not enabled:
            return
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(variants):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        step_fn(i)
                    self.graphs.append(g)
                size = min(self.GROUP, variants)
                for first in range(0, variants - size + 1, size) if size > 1 else ():
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=side):
                        for i in range(first, first + size):
                            step_fn(i)
                    self.groups[first] = (g, size)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            self.mode = "cuda_graph" if not self.groups else "cuda_graph (%d steps per replay)" % min(self.GROUP, variants)
        except Exception as exc:  # keep measuring, but say how
            self.graphs, self.groups, self.mode = [], {}, f"direct (graph capture failed: {type(exc).__name__})"
            torch.cuda.synchronize()

    def __call__(self, i: int):
        if self.graphs:
            self.graphs[i % len(self.graphs)].replay()
        else:
            self.step_fn(i)

    def run_many(self, start: int, count: int):
        """Steps start .. start + count - 1: whole groups from the group graphs, the rest one by one."""
        i, end = start, start + count
        while i < end:
            g, size = self.groups.get(i % len(self.graphs), (None, 0)) if self.graphs else (None, 0)
            if g is not None and end - i >= size:
                g.replay()
                i += size
            else:
                self(i)
                i += 1


def within_tolerance(got, want):
    """The tolerance of the parity tests: |a - b| <= 2e-3 + 1e-2 |b|.  Returns (ok, worst excess)."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    if not bool(torch.isfinite(got).all()):
        return False, float("inf")
    excess = float(((got - want).abs() - (2e-3 + 1e-2 * want.abs())).max())
    return excess <= 0, excess


# ------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------
def unit_pairs(q_lo, q_hi, window=None):
    """(query, visible key) pairs of the query positions [q_lo, q_hi): position p sees p + 1 keys,
    or the last ``window`` of them."""
    tri = lambda n: n * (n + 1) // 2
    if window is None:
        return tri(q_hi) - tri(q_lo)
    ramp_hi = min(q_hi, window)
    ramp = tri(ramp_hi) - tri(q_lo) if q_lo < ramp_hi else 0
    return ramp + (q_hi - max(q_lo, window)) * window if q_hi > window else ramp


def prefill_flops(B, S, window=None, heads=H):
    if window is None:
        pairs = S * (S + 1) // 2
    else:
        pairs = window * (window + 1) // 2 + (S - window) * window
    return 4.0 * B * heads * D * pairs


class PrefillWorkload:
    """Configs 2 and 3: q [B,S,H,D] physical (passed as the [B,H,S,D] view), caches [B,G,S,D].

    ``units`` (strong scaling over N > 1 GPUs) replaces the whole batch by this rank's share of
    it: a list of (request, kv head, q_lo, q_hi, k_lo) from dist.shard_prefill_units.  Every unit
    becomes one batch item with H/G query heads and one kv head, its queries the last
    q_hi - q_lo positions of the q_hi - k_lo keys it holds."""

    def __init__(self, name, dev, seed, units=None, full_batch=None):
        from g4b_b200.kernels import fa2

        self.fa2 = fa2
        self.name = name
        self.B, self.S, self.window = (4, 8192, None) if name.startswith("prefill_causal") else (2, 32768, 512)
        if full_batch is not None:
            self.B = full_batch
        self.dtype = torch.bfloat16
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.total_units = prefill_flops(self.B, self.S, self.window)      # whole job, FLOPs per step
        self.scaling = "weak"
        if units is None:
            B, Hh, Gg, Tq, Tk = self.B, H, G, self.S, self.S
            self.units = self.total_units
        else:
            assert len({(u[3] - u[2], u[3] - u[4]) for u in units}) == 1, "units of one rank must have one shape"
            B, Hh, Gg = len(units), H // G, 1
            Tq, Tk = units[0][3] - units[0][2], units[0][3] - units[0][4]
            self.units = sum(4.0 * Hh * D * unit_pairs(u[2], u[3], self.window) for u in units)
            self.scaling = "strong"
        self.Bl, self.Hl, self.Gl, self.Tq, self.Tk = B, Hh, Gg, Tq, Tk
        # pinned host copies: source of the e2e leg's per-step uploads
        self.h_q = torch.randn(B, Tq, Hh, D, generator=gen).to(self.dtype).pin_memory()
        self.h_k = torch.randn(B, Gg, Tk, D, generator=gen).to(self.dtype).pin_memory()
        self.h_v = torch.randn(B, Gg, Tk, D, generator=gen).to(self.dtype).pin_memory()
        self.h_o = torch.empty(B, Tq, Hh, D, dtype=self.dtype).pin_memory()
        self.q, self.k, self.v = self.h_q.to(dev), self.h_k.to(dev), self.h_v.to(dev)
        self.o = torch.empty_like(self.q)
        self.time = torch.full((B,), Tk, dtype=torch.int32, device=dev)
        self.metric, self.unit, self.bound, self.div = "prefill_attn_tflops", "TFLOP/s", "tensor", 1e12
        self.launches_per_step = 1
        self.h2d = (self.h_q.numel() + self.h_k.numel() + self.h_v.numel()) * 2
        self.d2h = self.h_o.numel() * 2
        self.config = {"workload": name, "batch_per_gpu": self.B, "seq_len": self.S, "q_heads": H, "kv_heads": G,
                       "head_dim": D, "window": self.window, "scale": SCALE,
                       "l2": "inputs (%d MB) larger than L2" % ((self.h2d + self.d2h) >> 20)}
        if units is not None:
            del self.config["batch_per_gpu"]
            self.config.update({"batch": self.B, "units_this_rank": [list(u) for u in units],
                                "unit_shape": {"q_heads": Hh, "kv_heads": Gg, "q_rows": Tq, "keys": Tk}})

    variants = 1

    def step(self, i=0):
        self.fa2.flash_attention(self.q.permute(0, 2, 1, 3), self.k, self.v, self.o.permute(0, 2, 1, 3), self.time,
                                 None, self.Tk, self.fa2.PHASE_PREFILL, scale=SCALE, sliding_window=self.window)

    def parity(self):
        """Sampled query rows of the first and the last batch item against the oracle."""
        from oracle import attention_oracle as orc

        self.step(0)
        torch.cuda.synchronize()
        ok, worst = True, -1.0
        for b in sorted({0, self.Bl - 1}):
            k, v = self.h_k[b].float(), self.h_v[b].float()
            for r in sorted({0, 1, self.Tq // 2 + 77, self.Tq - 1}):
                pos = self.Tk - self.Tq + r
                want = orc.attention_core(self.h_q[b, r:r + 1].float().permute(1, 0, 2), k[:, :pos + 1], v[:, :pos + 1],
                                          scale=SCALE, causal=True, sliding_window=self.window)
                good, ex = within_tolerance(self.o[b, r:r + 1].permute(1, 0, 2), want)
                ok, worst = ok and good, max(worst, ex)
        return ok, worst

    # End-to-end leg: a three-stage pipeline over two device buffer sets -- upload of step
    # i+1 (copy stream), attention of step i (launching stream) and download of step i-1
    # (second copy stream) overlap; PCIe is full duplex.  Every step still uploads its own
    # q / k / v from pinned memory and downloads its own o.
    def e2e_begin(self):
        dev = self.q.device
        self.s_up, self.s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        self.sets = [(self.q, self.k, self.v, self.o),
                     (torch.empty_like(self.q), torch.empty_like(self.k), torch.empty_like(self.v),
                      torch.empty_like(self.o))]
        self.ev_up = [torch.cuda.Event() for _ in range(2)]
        self.ev_done = [torch.cuda.Event() for _ in range(2)]
        self.ev_down = [torch.cuda.Event() for _ in range(2)]
        self.used = [False, False]
        cur = torch.cuda.current_stream()
        self.s_up.wait_stream(cur)
        self.s_down.wait_stream(cur)

    def e2e_step(self, i=0):
        b = i % 2
        q, k, v, o = self.sets[b]
        cur = torch.cuda.current_stream()
        with torch.cuda.stream(self.s_up):
            if self.used[b]:
                self.s_up.wait_event(self.ev_done[b])       # the kernel that read this set is done
            q.copy_(self.h_q, non_blocking=True)
            k.copy_(self.h_k, non_blocking=True)
            v.copy_(self.h_v, non_blocking=True)
            self.ev_up[b].record(self.s_up)
        cur.wait_event(self.ev_up[b])
        if self.used[b]:
            cur.wait_event(self.ev_down[b])                 # o of this set has been downloaded
        self.fa2.flash_attention(q.permute(0, 2, 1, 3), k, v, o.permute(0, 2, 1, 3), self.time, None, self.Tk,
                                 self.fa2.PHASE_PREFILL, scale=SCALE, sliding_window=self.window)
        self.ev_done[b].record(cur)
        with torch.cuda.stream(self.s_down):
            self.s_down.wait_event(self.ev_done[b])
            self.h_o.copy_(o, non_blocking=True)
            self.ev_down[b].record(self.s_down)
        self.used[b] = True

    def e2e_end(self):
        cur = torch.cuda.current_stream()
        cur.wait_stream(self.s_down)
        cur.wait_stream(self.s_up)

    def copy_ceiling(self, world, dev, reps=4):
        """What the e2e leg's own pinned buffers reach with copies alone, all ranks at once:
        uploads only, downloads only (GB/s per rank, from the slowest rank's time).  The e2e leg
        overlaps the two directions, so its floor per step is the slower of the two."""
        out = {}
        for key, pairs, nbytes in (("h2d", [(self.q, self.h_q), (self.k, self.h_k), (self.v, self.h_v)], self.h2d),
                                   ("d2h", [(self.h_o, self.o)], self.d2h)):
            def once(_i=0):
                for dst, src in pairs:
                    dst.copy_(src, non_blocking=True)
            ms = timed_region(once, reps, 2, world, dev) / reps
            out[key + "_gbs_per_rank"] = round(nbytes / (ms * 1e-3) / 1e9, 2)
            out[key + "_ms_per_step"] = round(ms, 4)
        out["e2e_floor_ms_per_step"] = max(out["h2d_ms_per_step"], out["d2h_ms_per_step"])
        out["ranks_copying_at_once"] = world
        return out

    def cpu_sample(self, budget_s=15.0):
        """Oracle on host cores: whole batch items, all heads, in 1024-query blocks, while the
        budget lasts.  Returns (TFLOP/s, description)."""
        from oracle import attention_oracle as orc

        q = self.h_q.float().permute(0, 2, 1, 3)
        k, v = self.h_k.float(), self.h_v.float()
        S = self.Tk if self.window is None else min(self.Tk, 8192)     # bounded sample of the long SWA sequence
        done, t0 = 0, time.perf_counter()
        while done < self.Bl and (done == 0 or time.perf_counter() - t0 < budget_s / 2):
            orc.attention_core(q[done][:, :S], k[done][:, :S], v[done][:, :S], scale=SCALE, causal=True,
                               sliding_window=self.window)
            done += 1
        dt = time.perf_counter() - t0
        flops = prefill_flops(done, S, self.window, heads=self.Hl)
        return flops / dt / 1e12, f"{done} of {self.Bl} batch items, first {S} tokens, fp32, 1024-query blocks"


class PrefillChunkWorkload:
    """One request's prefill chunk late in a long context: 256 new rows attend to 65536 cached
    keys (B1 H16 G4 D256 bf16, ring cache, causal) -- the shape of the reference's own
    prefill_t256_w65536 comparison case.  Only 32 (head, 128-row tile) units: the kernel splits
    their key ranges over the SMs (partial buffers given) and merges."""

    variants = 1
    scaling = "weak"

    def __init__(self, name, dev, seed, split=True):
        from g4b_b200.kernels import fa2

        self.fa2, self.name, self.dtype = fa2, name, torch.bfloat16
        B, Hc, Gc, t, T = 1, 16, 4, 256, 65536
        self.B, self.t, self.T, self.Hc = B, t, T, Hc
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.h_q = torch.randn(B, t, Hc, D, generator=gen).to(self.dtype).pin_memory()
        self.h_o = torch.empty(B, t, Hc, D, dtype=self.dtype).pin_memory()
        gdev = torch.Generator(device=dev).manual_seed(seed + 1)
        self.k = torch.randn(B, Gc, T, D, generator=gdev, device=dev, dtype=torch.float32).to(self.dtype)
        self.v = torch.randn(B, Gc, T, D, generator=gdev, device=dev, dtype=torch.float32).to(self.dtype)
        self.q = self.h_q.to(dev)
        self.o = torch.empty_like(self.q)
        self.time = torch.full((B,), T, dtype=torch.int32, device=dev)
        S = 16 if split else 0
        self.po = torch.empty(S, B, Hc, t, D, device=dev) if split else None
        self.pl = torch.empty(S, B, Hc, t, device=dev) if split else None
        self.pm = torch.empty(S, B, Hc, t, device=dev) if split else None
        self.units = 4.0 * B * Hc * D * (t * (T - t) + t * (t + 1) / 2)
        self.total_units = None
        self.metric, self.unit, self.bound, self.div = "prefill_attn_tflops", "TFLOP/s", "tensor", 1e12
        self.launches_per_step = 2 if split else 1
        self.h2d, self.d2h = self.h_q.numel() * 2, self.h_o.numel() * 2
        self.config = {"workload": name, "batch_per_gpu": B, "chunk_rows": t, "context": T, "q_heads": Hc, "kv_heads": Gc,
                       "head_dim": D, "scale": SCALE, "split_kv": bool(split),
                       "l2": "K/V (%d MB) larger than L2" % ((self.k.numel() + self.v.numel()) * 2 >> 20)}

    def step(self, i=0):
        self.fa2.flash_attention(self.q.permute(0, 2, 1, 3), self.k, self.v, self.o.permute(0, 2, 1, 3), self.time, None,
                                 self.T, self.fa2.PHASE_PREFILL, self.po, self.pl, self.pm, scale=SCALE)

    def e2e_step(self, i=0):
        self.q.copy_(self.h_q, non_blocking=True)
        self.step(i)
        self.h_o.copy_(self.o, non_blocking=True)

    def cpu_sample(self, budget_s=15.0):
        from oracle import attention_oracle as orc

        n = 32     # rows of the chunk
        q = self.h_q[0, :n].float().permute(1, 0, 2)
        k, v = self.k[0].float().cpu(), self.v[0].float().cpu()
        t0 = time.perf_counter()
        orc.attention_core(q, k[:, : self.T - self.t + n], v[:, : self.T - self.t + n], scale=SCALE, causal=True)
        dt = time.perf_counter() - t0
        return 4.0 * self.Hc * D * n * (self.T - self.t + n / 2) / dt / 1e12, f"{n} of {self.t} chunk rows, all heads, fp32"


class RopeAppendWorkload:
    """The launch right before attention on a prefill chunk: per-head RMS norm + rotary
    embedding of q and k, V norm, append of k and v to the ring caches, q out in bf16.  fp32
    inputs in the engine's [B,t,heads,D] layout (B4 t8192 H8 G2 D256), bf16 caches.  HBM-bound:
    algorithmic bytes = fp32 reads of q, k, v + bf16 writes of q, k, v."""

    variants = 1
    scaling = "weak"

    def __init__(self, name, dev, seed):
        from g4b_b200.kernels.rope import rope_norm_append

        self.fn = rope_norm_append
        self.name, self.dtype = name, torch.bfloat16
        B, S = 4, 8192
        self.B, self.S = B, S
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.h_q = torch.randn(B, S, H, D, generator=gen).pin_memory()
        self.h_k = torch.randn(B, S, G, D, generator=gen).pin_memory()
        self.h_v = torch.randn(B, S, G, D, generator=gen).pin_memory()
        self.q, self.k, self.v = self.h_q.to(dev), self.h_k.to(dev), self.h_v.to(dev)
        self.q16 = torch.empty(B, S, H, D, dtype=self.dtype, device=dev)
        self.h_q16 = torch.empty(B, S, H, D, dtype=self.dtype).pin_memory()
        self.kc = torch.zeros(B, G, S, D, dtype=self.dtype, device=dev)
        self.vc = torch.zeros(B, G, S, D, dtype=self.dtype, device=dev)
        self.qw = (1 + 0.1 * torch.randn(D, generator=gen)).to(dev)
        self.kw = (1 + 0.1 * torch.randn(D, generator=gen)).to(dev)
        self.freqs = (1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))).to(dev)
        self.off = torch.zeros(B, dtype=torch.int32, device=dev)
        rows = B * S
        self.units = float(rows * (H + 2 * G) * D * (4 + 2))
        self.total_units = None
        self.metric, self.unit, self.bound, self.div = "rope_append_hbm_gbs", "GB/s", "hbm", 1e9
        self.launches_per_step = 1
        self.h2d = (self.h_q.numel() + self.h_k.numel() + self.h_v.numel()) * 4
        self.d2h = self.h_q16.numel() * 2
        self.config = {"workload": name, "batch_per_gpu": B, "tokens": S, "q_heads": H, "kv_heads": G, "head_dim": D,
                       "in_dtype": "f32", "out_dtype": "bf16", "l2": "inputs (%d MB) larger than L2" % (self.h2d >> 20)}

    def step(self, i=0):
        self.fn(self.q.permute(0, 2, 1, 3), self.k.permute(0, 2, 1, 3), self.v.permute(0, 2, 1, 3), self.freqs, self.off,
                self.kc, self.vc, 1e-6, q_out=self.q16.permute(0, 2, 1, 3), q_rmsnorm_w=self.qw, k_rmsnorm_w=self.kw)

    def e2e_step(self, i=0):
        self.q.copy_(self.h_q, non_blocking=True)
        self.k.copy_(self.h_k, non_blocking=True)
        self.v.copy_(self.h_v, non_blocking=True)
        self.step(i)
        self.h_q16.copy_(self.q16, non_blocking=True)

    def cpu_sample(self, budget_s=15.0):
        from oracle import attention_oracle as orc

        n = 1024
        q, k, v = (x[:1, :n].permute(0, 2, 1, 3) for x in (self.h_q, self.h_k, self.h_v))
        kc, vc = torch.zeros(1, G, n, D, dtype=self.dtype), torch.zeros(1, G, n, D, dtype=self.dtype)
        t0 = time.perf_counter()
        orc.rope_norm_append(q, k, v, self.freqs.cpu(), torch.zeros(1, dtype=torch.int32), kc, vc, 1e-6,
                             q_rmsnorm_w=self.qw.cpu(), k_rmsnorm_w=self.kw.cpu())
        dt = time.perf_counter() - t0
        return n * (H + 2 * G) * D * 6 / dt / 1e9, f"{n} tokens of 1 batch item, torch fp32"


class KVAppendWorkload:
    """add_kv_to_cache on its own at prefill-chunk sizes: V rows [B,G,t,D] in fp32 with their
    precomputed sums of squares, normalised and cast into an f16 ring cache (B8 G4 t32768
    D256).  HBM-bound: algorithmic bytes = fp32 reads + f16 writes of the rows."""

    variants = 1
    scaling = "weak"

    def __init__(self, name, dev, seed):
        from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache

        self.fn, self.name, self.dtype = add_kv_to_cache, name, torch.float16
        B, S, Gk = 8, 32768, 4
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.h_x = torch.randn(B, S, Gk, D, generator=gen).pin_memory()       # the engine's [B,t,heads,D] layout
        self.x = self.h_x.to(dev)
        self.rsos = (self.x.permute(0, 2, 1, 3) ** 2).sum(-1)
        self.cache = torch.zeros(B, Gk, S, D, dtype=self.dtype, device=dev)
        self.h_probe = torch.empty(B, Gk, 16, D, dtype=self.dtype).pin_memory()
        self.d_probe = torch.empty(B, Gk, 16, D, dtype=self.dtype, device=dev)
        self.off = torch.zeros(B, dtype=torch.int32, device=dev)
        self.units = float(B * S * Gk * D * (4 + 2))
        self.total_units = None
        self.metric, self.unit, self.bound, self.div = "kv_append_hbm_gbs", "GB/s", "hbm", 1e9
        self.launches_per_step = 1
        self.h2d = self.h_x.numel() * 4
        self.d2h = self.h_probe.numel() * 2
        self.config = {"workload": name, "batch_per_gpu": B, "tokens": S, "kv_heads": Gk, "head_dim": D,
                       "in_dtype": "f32", "cache_dtype": "f16", "norm": True,
                       "l2": "inputs (%d MB) larger than L2" % (self.h2d >> 20)}

    def step(self, i=0):
        self.fn(self.x.permute(0, 2, 1, 3), self.cache, self.off, 1e-6, self.rsos)

    def e2e_step(self, i=0):
        self.x.copy_(self.h_x, non_blocking=True)
        self.step(i)
        self.d_probe.copy_(self.cache[:, :, :16])                         # the rows a caller would check
        self.h_probe.copy_(self.d_probe, non_blocking=True)

    def cpu_sample(self, budget_s=15.0):
        from oracle import attention_oracle as orc

        n = 2048
        x = self.h_x[:1, :n].permute(0, 2, 1, 3)
        cache = torch.zeros(1, x.shape[1], n, D, dtype=self.dtype)
        t0 = time.perf_counter()
        orc.add_kv_to_cache(x, cache, torch.zeros(1, dtype=torch.int32), 1e-6, (x ** 2).sum(-1))
        dt = time.perf_counter() - t0
        return n * x.shape[1] * D * 6 / dt / 1e9, f"{n} tokens of 1 batch item, torch fp32"


class DecodeWorkload:
    """Configs 4 and 5: paged KV with shuffled block tables; a step appends the new token's
    K and V rows and runs decode attention (split-KV + combine).

    decode_paged with ``shard`` on N > 1 GPUs: ONE set of sequences, dealt over the ranks
    longest-first (dist.balance_sequences); a rank holds only its sequences' pages.
    decode_long on N > 1 GPUs: the one sequence's pages are split contiguously over the ranks
    (dist.split_pages); its K/V values come from one seed, so that every rank's share belongs
    to the same sequence and the merged output can be checked against the oracle."""

    def __init__(self, name, dev, seed, rank=0, world=1, sequences=256, nccl_gather=False, kv_splits=0, shard=False,
                 fused=True, self_exchange=False):
        from g4b_b200 import dist as gdist
        from g4b_b200.kernels import fa2
        from g4b_b200.kernels.rope import rope_norm_append

        from g4b_b200.kernels.add_kv_to_cache import add_kv_to_cache_fp8

        self.fa2, self.append, self.append_fp8 = fa2, rope_norm_append, add_kv_to_cache_fp8
        self.name, self.dev, self.rank, self.world = name, dev, rank, world
        self.fused = fused      # the whole step as one launch (decode_step) or as append + decode + merge
        # with peers the merge and the exchange are inside the attention launch; --self-exchange runs
        # that form on one GPU (pushing to itself), to time the in-launch merge without a link
        self.merge_in_launch = (name == "decode_long" and world > 1) or self_exchange
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self.scaling = "weak"
        self.fp8 = name == "decode_paged_fp8"
        if name in ("decode_paged", "decode_paged_fp8"):
            self.dtype = torch.float16
            self.all_lens = torch.randint(1024, 32769, (sequences,), generator=gen, dtype=torch.int64)
            self.lens = self.all_lens
            self.splits = 16
            if shard and world > 1:
                mine = gdist.balance_sequences(self.all_lens.tolist(), world)[rank]
                self.lens = self.all_lens[mine]
                self.scaling = "strong"
        else:
            self.dtype = torch.bfloat16
            self.all_lens = self.lens = torch.tensor([131072], dtype=torch.int64)
            self.splits = 148          # x 2 kv heads = two CTAs on every SM
        self.long_split = name == "decode_long" and world > 1
        lens = self.lens
        B = len(lens)
        self.B = B
        pages_per = (lens + PAGE - 1) // PAGE
        if self.long_split:
            # this rank holds (and is handed block-table entries for) only its page range
            self.page_range = gdist.split_pages(int(pages_per[0]), world, rank)
            local_pages = torch.tensor([len(self.page_range)])
            self.local_lens = torch.tensor([min(int(lens[0]), self.page_range.stop * PAGE) - self.page_range.start * PAGE])
            self.splits = 128
            self.scaling = "strong"
        else:
            self.page_range = range(0, int(pages_per[0])) if name == "decode_long" else None
            local_pages, self.local_lens = pages_per, lens
        if kv_splits > 0:
            self.splits = kv_splits
        num_pages = int(local_pages.sum())
        perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(seed + 7 + rank)).to(torch.int32)
        if name == "decode_long":
            # the whole sequence from one seed on every rank; a rank keeps its page range, page i
            # of the range stored at pool position perm[i]
            gseq = torch.Generator(device=dev).manual_seed(seed + 1)
            L = int(lens[0])
            self.seq_k = self._big_randn((G, L, D), gseq)          # [G, L, D]
            self.seq_v = self._big_randn((G, L, D), gseq)
            lo, n = self.page_range.start * PAGE, len(self.page_range)
            def to_pool(seq):
                pages = seq[:, lo:lo + n * PAGE].reshape(G, n, PAGE, D).permute(1, 0, 2, 3)
                pool = torch.empty(n, G, PAGE, D, device=dev, dtype=self.dtype)
                pool[perm.to(dev).long()] = pages
                return pool
            self.k_pool, self.v_pool = to_pool(self.seq_k), to_pool(self.seq_v)
            if rank != 0:
                self.seq_k = self.seq_v = None                     # only rank 0 computes the oracle
        elif self.fp8:
            # bytes of finite e4m3 values (0x7f / 0xff are NaN) and scales as an append would leave them
            gdev = torch.Generator(device=dev).manual_seed(seed + 1 + rank)
            def bytes_pool():
                mag = torch.randint(0, 0x7f, (num_pages, G, PAGE, D), generator=gdev, device=dev, dtype=torch.int16)
                sign = torch.randint(0, 2, (num_pages, G, PAGE, D), generator=gdev, device=dev, dtype=torch.int16) << 7
                return (mag | sign).to(torch.uint8)
            self.k_pool, self.v_pool = bytes_pool(), bytes_pool()
            self.k_sc = 0.004 + 0.004 * torch.rand(num_pages, G, generator=gdev, device=dev)
            self.v_sc = 0.004 + 0.004 * torch.rand(num_pages, G, generator=gdev, device=dev)
        else:
            gdev = torch.Generator(device=dev).manual_seed(seed + 1 + rank)
            self.k_pool = self._big_randn((num_pages, G, PAGE, D), gdev)
            self.v_pool = self._big_randn((num_pages, G, PAGE, D), gdev)
        max_pages = int(local_pages.max())
        bt = torch.zeros(B, max_pages, dtype=torch.int32)
        at = 0
        for b in range(B):
            n = int(local_pages[b])
            bt[b, :n] = perm[at:at + n]
            at += n
        self.h_bt = bt
        self.bt = bt.to(dev)
        self.max_len = max_pages * PAGE
        self.time = self.local_lens.to(torch.int32).to(dev)
        self.off = (self.local_lens - 1).to(torch.int32).to(dev)
        gq = torch.Generator().manual_seed(seed + 3 + (0 if name == "decode_long" else rank))
        self.h_q = torch.randn(B, H, 1, D, generator=gq).to(self.dtype).pin_memory()
        self.h_kn = torch.randn(B, G, 1, D, generator=gq).to(self.dtype).pin_memory()
        self.h_vn = torch.randn(B, G, 1, D, generator=gq).to(self.dtype).pin_memory()
        self.h_o = torch.empty(B, H, 1, D, dtype=self.dtype).pin_memory()
        self.q, self.kn, self.vn = self.h_q.to(dev), self.h_kn.to(dev), self.h_vn.to(dev)
        self.o = torch.empty_like(self.q)
        S = self.splits
        self.packed = torch.empty(S, B, H, 1, D + 2, device=dev, dtype=torch.float32)
        self.po, self.pl, self.pm = self.packed[..., :D], self.packed[..., D], self.packed[..., D + 1]
        self.nccl_gather = nccl_gather
        self.exchange = None
        if self_exchange and world == 1:
            from g4b_b200 import _cabi

            xb = torch.zeros(_cabi.load().g4b_exchange_buffer_bytes(1, B * H, D) // 8, dtype=torch.int64, device=dev)
            self.exchange = gdist.PartialExchange(B * H, D, peers=[xb], rank=0)
        if self.long_split:
            self.gathered = torch.empty(world * S, B, H, 1, D + 2, device=dev, dtype=torch.float32)
            self.exchange = gdist.PartialExchange(B * H, D, device=dev)
            if not fused:
                self.launches_per_step = 3 if self.rank == world - 1 else 2
        esz = 1 if self.fp8 else 2
        kv_bytes = float(self.local_lens.sum()) * G * D * 2 * esz
        self.units = kv_bytes                                    # K/V bytes per step (this rank)
        self.total_units = float(self.all_lens.sum()) * G * D * 2 * esz if self.scaling == "strong" else None
        self.metric, self.unit, self.bound, self.div = "decode_attn_hbm_gbs", "GB/s", "hbm", 1e9
        # one launch; or append + attention, then the merge; or append (K and V), decode, merge
        self.launches_per_step = 4 if self.fp8 else ((1 if self.merge_in_launch else 2) if fused else 3)
        self.h2d = (self.h_q.numel() + self.h_kn.numel() + self.h_vn.numel()) * 2
        self.d2h = self.h_o.numel() * 2
        self.config = {"workload": name, "sequences": len(self.all_lens), "ctx_sum": int(self.all_lens.sum()),
                       "ctx_min": int(self.all_lens.min()), "ctx_max": int(self.all_lens.max()), "page_size": PAGE,
                       "kv_dtype": "e4m3 + f32 scale per (page, kv head)" if self.fp8 else str(self.dtype).replace("torch.", ""),
                       "kv_splits": self.splits, "scale": SCALE,
                       "l2": "K/V (%d MB per GPU) larger than L2" % (int(kv_bytes) >> 20)}
        if self.scaling == "strong":
            self.config.update({"sequences_this_rank": B, "ctx_sum_this_rank": int(self.local_lens.sum())})
        self.config["step"] = ("one launch (append + attention + merge + exchange)" if self.merge_in_launch else
                               "two launches (append + attention, merge)") if fused else "three launches (append, attention, merge)"
        if self.fp8:
            self.config["step"] = "four launches (K rows quantised into their pages, V rows, attention, merge)"
        if self.long_split:
            self.config["merge"] = "all-gather + second merge launch (NCCL)" if nccl_gather else \
                "inside the launch: local merge, exchange through peer memory, final merge"
        # a K/V set that is not several times the 126 MB L2 would be served from cache on the
        # next step: rotate over copies (same block table, distinct memory) totalling >= 1 GB
        self.pools = [(self.k_pool, self.v_pool)]
        if kv_bytes < 1e9:
            copies = int(math.ceil(1e9 / max(kv_bytes, 1.0)))
            for _ in range(copies - 1):
                self.pools.append((self.k_pool.clone(), self.v_pool.clone()))
            self.config["l2"] = "K/V %d MB per GPU: %d distinct copies used in rotation (> 1 GB)" % (
                int(kv_bytes) >> 20, len(self.pools))
        self.variants = len(self.pools)

    def _big_randn(self, shape, gdev):
        """N(0,1) values of the cache dtype, generated in chunks so that the fp32 temporary stays small."""
        out = torch.empty(shape, device=self.dev, dtype=self.dtype)
        flat = out.view(-1)
        chunk = 1 << 26
        for s in range(0, flat.numel(), chunk):
            e = min(flat.numel(), s + chunk)
            flat[s:e] = torch.randn(e - s, generator=gdev, device=self.dev, dtype=torch.float32).to(self.dtype)
        return out

    def step(self, i=0):
        self.k_pool, self.v_pool = self.pools[i % len(self.pools)]
        if self.fp8:
            # the new token's K and V rows are quantised into their pages, then attention over the bytes
            self.append_fp8(self.kn, self.k_pool, self.k_sc, self.off, 1e-6, block_tables=self.bt, page_size=PAGE)
            self.append_fp8(self.vn, self.v_pool, self.v_sc, self.off, 1e-6, block_tables=self.bt, page_size=PAGE)
            self.fa2.flash_attention_fp8(self.q, self.k_pool, self.v_pool, self.k_sc, self.v_sc, self.o, self.time, None,
                                         self.max_len, self.fa2.PHASE_DECODE, self.po, self.pl, self.pm, scale=SCALE,
                                         block_tables=self.bt, page_size=PAGE, num_kv_splits=self.splits)
            return
        last = (not self.long_split) or self.rank == self.world - 1
        if self.fused and not self.nccl_gather:
            # the new token's row lives on the rank that owns the tail of the sequence
            self.fa2.decode_step(self.q, self.k_pool, self.v_pool, self.o, self.time, None, self.max_len,
                                 self.fa2.PHASE_DECODE, self.po, self.pl, self.pm,
                                 k_new=self.kn if last else None, v_new=self.vn if last else None,
                                 exchange=self.exchange, num_kv_splits=self.splits,
                                 scale=SCALE, block_tables=self.bt, page_size=PAGE)
            return
        if last:
            # K and V rows in one launch (no rotation, no norm: a plain append of both)
            self.append(self.q, self.kn, self.vn, None, self.off, self.k_pool, self.v_pool, 1e-6,
                        norm_qk=False, norm_v=False, block_tables=self.bt, page_size=PAGE)
        if not self.long_split:
            self.fa2.flash_attention(self.q, self.k_pool, self.v_pool, self.o, self.time, None, self.max_len,
                                     self.fa2.PHASE_DECODE, self.po, self.pl, self.pm, scale=SCALE,
                                     block_tables=self.bt, page_size=PAGE, num_kv_splits=self.splits)
            return
        from g4b_b200 import dist as gdist

        self.fa2.attention_decode_partials(self.q, self.k_pool, self.v_pool, self.o, self.time, None, self.max_len,
                                           self.fa2.PHASE_DECODE, self.po, self.pl, self.pm, self.splits, scale=SCALE,
                                           block_tables=self.bt, page_size=PAGE)
        if self.nccl_gather:
            # the library-collective form: all-gather every split's partial, one merge
            gdist.gather_packed(self.packed, out=self.gathered)
            go, gl, gm = gdist.unpack_gathered(self.gathered)
            self.fa2.combine_partials(go, gl, gm, self.o, self.world * self.splits)
        else:
            # one kernel: local merge, exchange through peer memory, final merge
            self.exchange.combine(self.po, self.pl, self.pm, self.o, self.splits)

    def parity(self):
        """decode_long: the merged output of every rank against the oracle's attention over the
        whole sequence (rank 0 computes it and broadcasts), for the peer-memory merge and, on
        N > 1 GPUs, for the all-gather merge too.  decode_paged: the first and the last local
        sequence against the oracle."""
        from oracle import attention_oracle as orc

        ok, worst = True, -1.0
        if self.name == "decode_long":
            want = torch.empty(1, H, 1, D, device=self.dev)
            if self.rank == 0:
                L = int(self.all_lens[0])
                k, v = self.seq_k.float().cpu(), self.seq_v.float().cpu()
                k[:, L - 1], v[:, L - 1] = self.h_kn[0, :, 0].float(), self.h_vn[0, :, 0].float()   # the appended row
                want.copy_(orc.attention_core(self.h_q[0].float(), k, v, scale=SCALE)[None])
                self.seq_k = self.seq_v = None
            if self.world > 1:
                torch.distributed.broadcast(want, 0)
            forms = [False, True] if self.long_split else [False]
            keep = self.nccl_gather
            for form in forms:
                self.nccl_gather = form
                self.o.zero_()
                self.step(0)
                torch.cuda.synchronize()
                good, ex = within_tolerance(self.o, want)
                ok, worst = ok and good, max(worst, ex)
            self.nccl_gather = keep
            return ok, worst
        self.step(0)
        torch.cuda.synchronize()
        kp, vp = self.pools[0]
        for b in sorted({0, self.B - 1}):
            L = int(self.local_lens[b])
            pages = self.h_bt[b, : (L + PAGE - 1) // PAGE].long()
            if self.fp8:
                k = orc.dequantise_fp8_pool(kp[pages.to(self.dev)].cpu(), self.k_sc[pages.to(self.dev)].cpu())
                v = orc.dequantise_fp8_pool(vp[pages.to(self.dev)].cpu(), self.v_sc[pages.to(self.dev)].cpu())
                k, v = (torch.nan_to_num(x).permute(1, 0, 2, 3).reshape(G, -1, D)[:, :L] for x in (k, v))
            else:
                k = kp[pages.to(self.dev)].float().cpu().permute(1, 0, 2, 3).reshape(G, -1, D)[:, :L]
                v = vp[pages.to(self.dev)].float().cpu().permute(1, 0, 2, 3).reshape(G, -1, D)[:, :L]
            want = orc.attention_core(self.h_q[b].float(), k, v, scale=SCALE)
            good, ex = within_tolerance(self.o[b], want)
            ok, worst = ok and good, max(worst, ex)
        return ok, worst

    def e2e_step(self, i=0):
        self.q.copy_(self.h_q, non_blocking=True)
        self.kn.copy_(self.h_kn, non_blocking=True)
        self.vn.copy_(self.h_vn, non_blocking=True)
        self.step(i)
        self.h_o.copy_(self.o, non_blocking=True)

    def cpu_sample(self, budget_s=15.0):
        from oracle import attention_oracle as orc

        n = min(8, self.B)
        idx = list(range(n))
        if self.fp8:     # the CPU side has no 8-bit path: it attends over the de-quantised values of the sample
            used = torch.unique(self.h_bt[:n].flatten().long().clamp(min=0)).to(self.dev)
            kp = torch.zeros(self.k_pool.shape, dtype=torch.float16)
            vp = torch.zeros(self.v_pool.shape, dtype=torch.float16)
            kp[used.cpu()] = torch.nan_to_num(orc.dequantise_fp8_pool(self.k_pool[used].cpu(), self.k_sc[used].cpu())).half()
            vp[used.cpu()] = torch.nan_to_num(orc.dequantise_fp8_pool(self.v_pool[used].cpu(), self.v_sc[used].cpu())).half()
        else:
            kp, vp = self.k_pool.cpu(), self.v_pool.cpu()
        t0 = time.perf_counter()
        touched = 0
        for b in idx:
            L = int(self.local_lens[b])
            k = orc.gather_pages(kp, self.h_bt[b], L, PAGE)
            v = orc.gather_pages(vp, self.h_bt[b], L, PAGE)
            orc.attention_core(self.h_q[b].float(), k, v, scale=SCALE)
            touched += L * G * D * 2 * (1 if self.fp8 else 2)
        dt = time.perf_counter() - t0
        return touched / dt / 1e9, f"{n} of {self.B} sequences ({touched >> 20} MB of K/V), page gather + fp32 attention"


def make_workload(name, dev, rank, world, sequences=256, nccl_gather=False, kv_splits=0, strong=False, fused=True,
                  self_exchange=False):
    """``strong``: the workload is ONE job dealt over the ranks (strong scaling) instead of the
    same per-GPU batch on every rank."""
    from g4b_b200 import dist as gdist

    seeds = {"prefill_causal": 1, "prefill_swa": 2, "decode_paged": 3, "decode_long": 4, "rope_append": 5,
             "kv_append": 7, "decode_paged_fp8": 3}
    if name == "kv_append":
        return KVAppendWorkload(name, dev, seeds[name] + 100 * rank)
    if name == "rope_append":
        return RopeAppendWorkload(name, dev, seeds[name] + 100 * rank)
    if name == "prefill_chunk":
        return PrefillChunkWorkload(name, dev, 6 + 100 * rank, split=kv_splits >= 0)
    if name.startswith("prefill"):
        units = None
        if strong and world > 1:
            nreq, S, W = (4, 8192, None) if name == "prefill_causal" else (2, 32768, 512)
            units = gdist.shard_prefill_units(nreq, G, S, world, rank, W)
        return PrefillWorkload(name, dev, seeds[name] + 100 * rank, units=units)
    return DecodeWorkload(name, dev, seeds[name] + (0 if name == "decode_long" else 100 * rank), rank, world,
                          sequences, nccl_gather, kv_splits, shard=strong, fused=fused, self_exchange=self_exchange)


# ------------------------------------------------------------------------------------------
# arms
# ------------------------------------------------------------------------------------------
def value_of(wl, ms_step, world):
    """Whole-job throughput in the workload's unit: work of all ranks / time of the slowest."""
    total = wl.total_units if wl.scaling == "strong" and wl.total_units is not None else wl.units * world
    return total / (ms_step * 1e-3) / wl.div


def roofline_of(wl, value, world, peaks, sustained=False):
    peak = (peaks["tensor_sustained"] if sustained else peaks["tensor"]) if wl.bound == "tensor" else peaks["hbm"]
    per_gpu = value / world
    cap = captured_traffic(wl.name)
    traffic = None
    if cap is not None:     # per launch on one rank, scaled from the captured case by the units processed
        traffic = cap["dram_bytes_per_algorithmic_unit"] * wl.units + cap.get("dram_bytes_per_batch_item", 0.0) * getattr(wl, "B", 0)
    kind = ("sustained" if sustained else "burst") if wl.bound == "tensor" else "copy"
    return {"bound": wl.bound, "achieved": round(per_gpu, 3), "peak": peak, "unit": wl.unit,
            "frac": round(per_gpu / peak, 4), "traffic": traffic, "peak_source": f"{peaks['source']} {kind}"}


def measure(wl, steps, warmup, world, dev, use_graph, sampler=None):
    """Returns (ms per step: max over ranks, launch mode, the runner)."""
    for i in range(3):          # first calls set kernel attributes etc.: keep them out of capture
        wl.step(i)
    torch.cuda.synchronize()
    run = GraphRunner(wl.step, wl.variants, use_graph)
    ms = timed_region(run, steps, warmup, world, dev, sampler) / steps
    return ms, run.mode, run


def run_block(name, dev, rank, world, peaks, args, steps, warmup, *, strong, cpu=True):
    """One extra block of the default line: build the workload, check it against the oracle,
    time it, describe it."""
    wl = make_workload(name, dev, rank, world, strong=strong)
    good, excess = wl.parity()
    good = all_ranks_ok(good, world, dev)
    if not good:
        raise SystemExit(f"rank {rank}: {name}: output differs from the oracle (tolerance exceeded by {excess:.3e})")
    # a step that contains an NCCL collective is launched directly
    use_graph = not args.no_graph and not (getattr(wl, "long_split", False) and wl.nccl_gather)
    ms, mode, _ = measure(wl, steps, warmup, world, dev, use_graph)
    value = value_of(wl, ms, world)
    out = {"metric": wl.metric, "value": round(value, 2), "unit": wl.unit, "ms_per_step": round(ms, 5),
           "scaling": wl.scaling if world > 1 else "single GPU", "n_gpus": world, "steps": steps,
           "config": wl.config, "launch": mode, "roofline": roofline_of(wl, value, world, peaks),
           "parity": "ok", "parity_tolerance": "|a-b| <= 2e-3 + 1e-2|b| against the CPU oracle, all ranks",
           "gpu_launches": wl.launches_per_step * steps}
    if getattr(wl, "long_split", False):
        wl.nccl_gather = True
        wl.config = dict(wl.config)
        ms2, _, _ = measure(wl, steps, warmup, world, dev, False)
        out["nccl_all_gather_form_ms_per_step"] = round(ms2, 5)
    if cpu and rank == 0 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline_of(wl, world, args.no_cpu)
    return out


def cpu_leg_in_child(argv):
    """Under torchrun every rank starts with OMP_NUM_THREADS=1 and its BLAS initialised for one
    thread; raising the count afterwards oversubscribes instead of helping.  So a rank that wants
    a CPU leg with all cores runs it in a fresh interpreter without the launcher's variables and
    reads the JSON line that prints."""
    import subprocess

    env = {k: v for k, v in os.environ.items()
           if not (k.startswith(("OMP_", "MKL_", "TORCHELASTIC", "GROUP_", "ROLE_")) or k in (
               "RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"))}
    res = subprocess.run([sys.executable, str(ROOT / "bench.py"), *argv], env=env, capture_output=True, text=True, timeout=900)
    lines = [ln for ln in res.stdout.strip().splitlines() if ln.startswith("{")]
    if res.returncode != 0 or not lines:
        return {"unavailable": f"CPU leg exited {res.returncode}: {res.stderr.strip()[-200:]}"}
    return json.loads(lines[-1])


def cpu_baseline_of(wl, world, no_cpu):
    """The workload's CPU baseline block (one-GPU runs only)."""
    if no_cpu:
        return None
    if world > 1:
        # the other ranks spin in their barrier on the same cores: the CPU figure belongs to the one-GPU line
        return None
    v, sample = wl.cpu_sample()
    return {"value": round(v, 5), "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port", "sample": sample}


def cpu_config1():
    """Configuration 1, the reference's CPU case: B1 S512 H8 G2 D256 fp32 causal, scale 1/16,
    through the oracle on the host cores, timed in full (median of 7 warm runs)."""
    from oracle import attention_oracle as orc

    gen = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(h, 512, D, generator=gen) for h in (H, G, G))
    orc.attention_core(q, k, v, scale=SCALE)
    times = []
    for _ in range(7):
        t0 = time.perf_counter()
        orc.attention_core(q, k, v, scale=SCALE)
        times.append(time.perf_counter() - t0)
    dt = sorted(times)[len(times) // 2]
    flops = prefill_flops(1, 512)
    return {"workload": "B1 S512 H8 G2 D256 fp32 causal", "ms": round(dt * 1e3, 3), "gflops_causal": round(flops / dt / 1e9, 2),
            "gflops_as_executed_dense": round(2 * flops * 512 / 513 / dt / 1e9, 2), "cores": torch.get_num_threads(),
            "kind": "port", "runs": len(times)}


def bind_near_gpu(local):
    """Keeps this rank's threads (and so its first-touch pinned pages) on the CPUs NVML lists
    as near its GPU.  Changes only this process's affinity, no device setting."""
    info = {"affinity_before": sorted(os.sched_getaffinity(0))}
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = [64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1]
        allowed = sorted(set(cpus) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
        info["cpus_near_gpu"] = len(allowed)
    except Exception as exc:
        info["cpus_near_gpu"] = f"unknown ({type(exc).__name__})"
    try:
        info["numa_nodes"] = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node")])
    except Exception:
        info["numa_nodes"] = None
    return info


def run_ours(args):
    rank, world, local = dist_env()
    if args.gpus != world and world == 1 and args.gpus > 1:
        raise SystemExit("launch N > 1 with torchrun (one rank per GPU)")
    dev = torch.device(f"cuda:{local}")
    torch.cuda.set_device(dev)
    host = bind_near_gpu(local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    import __graft_entry__

    if rank == 0:
        __graft_entry__.build()
    if world > 1:
        torch.distributed.barrier()
    from g4b_b200 import _cabi

    peaks = measured_peaks()
    headline = args.workload == "prefill_causal" and not args.no_extras
    wl = make_workload(args.workload, dev, rank, world, args.sequences, args.nccl_gather, args.kv_splits,
                       strong=args.strong, fused=not args.unfused, self_exchange=args.self_exchange)
    parity = None
    if hasattr(wl, "parity"):
        good, excess = wl.parity()
        if not all_ranks_ok(good, world, dev):
            raise SystemExit(f"rank {rank}: {args.workload}: output differs from the oracle (tolerance exceeded by {excess:.3e})")
        parity = "ok"
    sampler = ClockSampler(local) if rank == 0 else None
    # a step that contains an NCCL collective is launched directly: replaying captured
    # collectives from several graphs stalled here
    use_graph = not args.no_graph and not (getattr(wl, "long_split", False) and args.nccl_gather)
    ms_step, mode, run_step = measure(wl, args.steps, args.warmup, world, dev, use_graph, sampler)
    clocks = sampler.stop() if sampler is not None else None
    value = value_of(wl, ms_step, world)

    # end to end: pinned host inputs -> device -> operators -> pinned host result, every step
    if hasattr(wl, "e2e_begin"):      # multi-stream pipeline, launched from Python
        ms_e2e = timed_region(wl.e2e_step, args.steps, args.warmup, world, dev,
                              begin=wl.e2e_begin, end=wl.e2e_end) / args.steps
    else:
        run_e2e = GraphRunner(wl.e2e_step, wl.variants, use_graph)
        ms_e2e = timed_region(run_e2e, args.steps, args.warmup, world, dev) / args.steps
    e2e_value = value_of(wl, ms_e2e, world)
    status = _cabi.device_status()
    if status != 0:
        raise SystemExit(f"device status word {status:#x}: a kernel gave up on a bounded wait")

    out = {
        "metric": wl.metric, "value": round(value, 3), "unit": wl.unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
        "scaling": wl.scaling, "vs_baseline": None,
        "dtype": "bf16" if wl.dtype == torch.bfloat16 else "f16", "data": "synthetic (seeded N(0,1))",
        "config": wl.config, "launch": mode,
        "e2e": {"value": round(e2e_value, 3), "unit": wl.unit, "h2d_bytes_per_step": wl.h2d,
                "d2h_bytes_per_step": wl.d2h, "ms_per_step": round(ms_e2e, 5)},
        "gpu_launches": wl.launches_per_step * args.steps,
        "roofline": roofline_of(wl, value, world, peaks),
        "clocks": clocks, "host": host,
    }
    if parity is not None:
        out["parity"] = parity
    if hasattr(wl, "copy_ceiling"):
        out["e2e"]["copy_ceiling"] = wl.copy_ceiling(world, dev)
    if headline or args.sustained:
        # the same step replayed back to back for about two seconds: what the kernel holds once
        # the power limit bites, beside the clock it ran at
        n = max(args.steps, int(2200.0 / ms_step))
        s2 = ClockSampler(local) if rank == 0 else None
        ms_s = timed_region(run_step, n, 3, world, dev, s2) / n
        c2 = s2.stop() if s2 is not None else None
        v2 = value_of(wl, ms_s, world)
        out["sustained"] = {"steps": n, "seconds": round(ms_s * n / 1e3, 2), "ms_per_step": round(ms_s, 5),
                            "value": round(v2, 3), "unit": wl.unit, "clocks": c2,
                            "ms_x_mhz": (round(ms_s * c2["sm_mhz"], 1) if c2 and c2["sm_mhz"] else None),
                            "roofline": roofline_of(wl, v2, world, peaks, sustained=True)}
    # the CPU legs get every core this process started with, not only those near the GPU
    os.sched_setaffinity(0, host.pop("affinity_before"))
    if rank == 0 and not args.no_cpu:
        out["cpu_baseline"] = cpu_baseline_of(wl, world, args.no_cpu)
    if headline:
        # the other configurations of the metric, each with its own oracle check
        del wl, run_step
        torch.cuda.empty_cache()
        k2, w2 = max(5, args.steps // 2), max(3, args.warmup)
        if world > 1:
            out["prefill_strong"] = run_block("prefill_causal", dev, rank, world, peaks, args, k2, w2, strong=True, cpu=False)
            torch.cuda.empty_cache()
        for key, name in (("swa", "prefill_swa"), ("decode", "decode_paged"), ("decode_fp8", "decode_paged_fp8"),
                          ("decode_long", "decode_long")):
            out[key] = run_block(name, dev, rank, world, peaks, args, k2, w2, strong=True)
            torch.cuda.empty_cache()
        status = _cabi.device_status()
        if status != 0:
            raise SystemExit(f"device status word {status:#x} after the extra blocks")
        if rank == 0 and not args.no_cpu:
            out["cpu_config1"] = cpu_config1() if world == 1 else None
        if rank == 0 and not args.no_triton:
            try:
                from baseline import triton_reference

                out["triton_reference"] = triton_reference.run(["prefill_causal", "decode_ring"], tuned=False, reps=3)
            except Exception as exc:       # informational block: never fail the line over it
                out["triton_reference"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    if world > 1:
        torch.distributed.barrier()
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        torch.distributed.destroy_process_group()


def reference_prefill_fn(q, k, v, window):
    """One pass over the batch with the reference's own LayerKVCache (scripts/reference_impl.py,
    loaded unmodified from the copies oracle/make_ref.py leaves beside the oracle), or None when
    they are not there.  q [B,H,S,D] fp32 pre-scaled, k / v [B,G,S,D] fp32."""
    try:
        from oracle import ref_loader

        if not ref_loader.available() or window is not None:
            return None          # the reference materialises [H,S,S] scores: 34 GB per item at S = 32768
        Bq, Hh, S, _ = q.shape

        def run():
            for b in range(Bq):
                cache = ref_loader.make_layer_cache(heads=Hh, kv_heads=k.shape[1], head_dim=D, context_length=S,
                                                    sliding_window=S, is_swa=False)
                cache.set_prefill()
                cache.add(k[b:b + 1], v[b:b + 1])
                cache.retrieve(q[b:b + 1])
        return run
    except Exception:
        return None


def run_reference(args):
    """The reference's CPU attention on the host cores over the whole per-GPU batch of the
    workload: its own torch code where that can run (kind "reference"), else the oracle port of
    the same arithmetic (kind "port").  Rank 0 only."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    name = args.workload

    # build the same inputs on the host only (no GPU needed for this arm)
    from oracle import attention_oracle as orc

    gen = torch.Generator().manual_seed(1)
    kind = "port"
    if name in ("prefill_causal", "prefill_swa"):
        Bf, S, window = (4, 8192, None) if name == "prefill_causal" else (2, 32768, 512)
        q = torch.randn(Bf, H, S, D, generator=gen).to(torch.bfloat16).float()
        k = torch.randn(Bf, G, S, D, generator=gen).to(torch.bfloat16).float()
        v = torch.randn(Bf, G, S, D, generator=gen).to(torch.bfloat16).float()
        units = prefill_flops(Bf, S, window)

        def port():
            for b in range(Bf):
                orc.attention_core(q[b], k[b], v[b], scale=SCALE, causal=True, sliding_window=window)

        fn = port
        sample = f"all {Bf} batch items x {S} tokens, all {H} heads per step, fp32, 1024-query blocks"
        ref_fn = reference_prefill_fn(q * SCALE, k, v, window)
        if ref_fn is not None and not args.port:
            t0 = time.perf_counter()
            ref_fn()
            probe = time.perf_counter() - t0
            if probe * (args.steps + args.warmup) < 420:       # keep the whole run within minutes
                fn, kind = ref_fn, "reference"
                sample = f"all {Bf} batch items x {S} tokens through the reference's LayerKVCache.add/.retrieve, fp32"
        metric, unit, div = "prefill_attn_tflops", "TFLOP/s", 1e12
        config = {"workload": name, "batch_per_gpu": Bf, "seq_len": S, "q_heads": H, "kv_heads": G,
                  "head_dim": D, "window": window, "scale": SCALE,
                  "l2": "inputs (%d MB) larger than L2" % ((2 * q.numel() + k.numel() + v.numel()) * 2 >> 20)}
    elif name == "prefill_chunk":
        Hc, Gc, t, T = 16, 4, 256, 65536
        q = torch.randn(Hc, t, D, generator=gen).to(torch.bfloat16).float()
        k = torch.randn(Gc, T, D, generator=gen).to(torch.bfloat16).float()
        v = torch.randn(Gc, T, D, generator=gen).to(torch.bfloat16).float()
        units = 4.0 * Hc * D * (t * (T - t) + t * (t + 1) / 2)
        fn = lambda: orc.attention_core(q, k, v, scale=SCALE, causal=True, q_block=32)
        metric, unit, div = "prefill_attn_tflops", "TFLOP/s", 1e12
        sample = f"all {t} chunk rows over {T} keys, all {Hc} heads per step, fp32, 32-query blocks"
        config = {"workload": name, "batch_per_gpu": 1, "chunk_rows": t, "context": T, "q_heads": Hc, "kv_heads": Gc,
                  "head_dim": D, "scale": SCALE}
    elif name == "rope_append":
        n = 1024
        q, k, v = (torch.randn(1, h, n, D, generator=gen) for h in (H, G, G))
        qw, kw = 1 + 0.1 * torch.randn(D, generator=gen), 1 + 0.1 * torch.randn(D, generator=gen)
        freqs = 1.0 / (10000.0 ** (torch.arange(0, D, 2) / D))
        kc, vc = torch.zeros(1, G, n, D, dtype=torch.bfloat16), torch.zeros(1, G, n, D, dtype=torch.bfloat16)
        off = torch.zeros(1, dtype=torch.int32)
        units = float(n * (H + 2 * G) * D * 6)
        fn = lambda: orc.rope_norm_append(q, k, v, freqs, off, kc, vc, 1e-6, q_rmsnorm_w=qw, k_rmsnorm_w=kw)
        metric, unit, div = "rope_append_hbm_gbs", "GB/s", 1e9
        sample = f"{n} tokens of 1 batch item per step, torch fp32"
        config = {"workload": name, "batch_per_gpu": 4, "tokens": 8192, "q_heads": H, "kv_heads": G, "head_dim": D,
                  "in_dtype": "f32", "out_dtype": "bf16", "reference_sample": sample}
    elif name == "kv_append":
        n, Gk = 2048, 4
        x = torch.randn(1, Gk, n, D, generator=gen)
        cache = torch.zeros(1, Gk, n, D, dtype=torch.float16)
        off = torch.zeros(1, dtype=torch.int32)
        units = float(n * Gk * D * 6)
        fn = lambda: orc.add_kv_to_cache(x, cache, off, 1e-6, (x ** 2).sum(-1))
        metric, unit, div = "kv_append_hbm_gbs", "GB/s", 1e9
        sample = f"{n} tokens of 1 batch item per step, torch fp32"
        config = {"workload": name, "batch_per_gpu": 8, "tokens": 32768, "kv_heads": Gk, "head_dim": D,
                  "in_dtype": "f32", "cache_dtype": "f16", "norm": True, "reference_sample": sample}
    else:
        # decode_paged: the first 8 sequences of the benchmark's seeded set (what the GPU arm's
        # cpu_baseline leg runs); decode_long: the one sequence
        if name in ("decode_paged", "decode_paged_fp8"):   # (the CPU side has no 8-bit path: same f16 sample)
            lens = torch.randint(1024, 32769, (256,), generator=torch.Generator().manual_seed(3), dtype=torch.int64)[:8]
            dt_kv = torch.float16
        else:
            lens, dt_kv = torch.tensor([131072]), torch.bfloat16
        pages = [(int(L) + PAGE - 1) // PAGE for L in lens]
        n_pages = sum(pages)
        kp = torch.randn(n_pages, G, PAGE, D, generator=gen).to(dt_kv)
        vp = torch.randn(n_pages, G, PAGE, D, generator=gen).to(dt_kv)
        perm = torch.randperm(n_pages, generator=gen).to(torch.int32)
        tables, at = [], 0
        for n in pages:
            tables.append(perm[at:at + n])
            at += n
        qs = torch.randn(len(lens), H, 1, D, generator=gen)
        units = float(lens.sum()) * G * D * 2 * 2

        def fn():
            for b, L in enumerate(lens):
                kk = orc.gather_pages(kp, tables[b], int(L), PAGE)
                vv = orc.gather_pages(vp, tables[b], int(L), PAGE)
                orc.attention_core(qs[b], kk, vv, scale=SCALE)

        metric, unit, div = "decode_attn_hbm_gbs", "GB/s", 1e9
        sample = f"{len(lens)} sequence(s), {int(lens.sum())} tokens per step, page gather + fp32 attention"
        config = {"workload": name, "sequences": 256 if name.startswith("decode_paged") else 1, "page_size": PAGE,
                  "kv_dtype": str(dt_kv).replace("torch.", ""), "scale": SCALE, "reference_sample": sample}
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    dt = (time.perf_counter() - t0) / args.steps
    value = units / dt / div
    out = {
        "impl": "reference", "metric": metric, "value": round(value, 5), "unit": unit, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic (seeded N(0,1))",
        "config": config,
        "cpu_baseline": {"value": round(value, 5), "unit": unit, "cores": torch.get_num_threads(), "kind": kind,
                         "sample": sample},
        "e2e": {"value": round(value, 5), "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="prefill_causal",
                    choices=["prefill_causal", "prefill_swa", "prefill_chunk", "decode_paged", "decode_long", "rope_append",
                             "kv_append", "decode_paged_fp8"])
    ap.add_argument("--sequences", type=int, default=256,
                    help="decode_paged only: number of sequences (256 = the benchmark configuration; "
                         "smaller values are for profiler captures)")
    ap.add_argument("--kv-splits", type=int, default=0, help="decode workloads: split count (0 = the workload's default); prefill_chunk: -1 = no split-KV")
    ap.add_argument("--nccl-gather", action="store_true",
                    help="decode_long on N > 1 GPUs: all-gather the partials with NCCL and merge in a second launch "
                         "instead of the one-kernel exchange over peer memory")
    ap.add_argument("--strong", action="store_true",
                    help="N > 1: deal ONE job over the ranks (prefill units, decode sequences) instead of the same batch on every rank")
    ap.add_argument("--unfused", action="store_true",
                    help="decode workloads: append, attention and merge as three launches instead of decode_step")
    ap.add_argument("--self-exchange", action="store_true",
                    help="decode workloads on one GPU: the one-launch form of decode_step (merge inside the launch, "
                         "pieces pushed to this GPU's own exchange buffer)")
    ap.add_argument("--no-graph", action="store_true", help="launch every step from Python instead of replaying CUDA graphs")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline legs")
    ap.add_argument("--no-extras", action="store_true", help="default workload: only the headline, none of the other configurations' blocks")
    ap.add_argument("--no-triton", action="store_true", help="default line: skip the reference's Triton kernel")
    ap.add_argument("--sustained", action="store_true", help="add the two-second replay to a single-workload line")
    ap.add_argument("--port", action="store_true", help="--impl reference: time the oracle port even where the reference's own torch code is present")
    ap.add_argument("--cpu-config1", action="store_true", help="only time configuration 1 on the host cores and print it")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.cpu_config1:
        torch.set_num_threads(os.cpu_count() or 1)
        print(json.dumps(cpu_config1()))
        return
    if args.impl == "reference":
        rank, world, _ = dist_env()
        if world > 1:
            # rank 0 alone measures, in a fresh interpreter with all host threads (see cpu_leg_in_child)
            if rank == 0:
                argv = ["--impl", "reference", "--workload", args.workload, "--steps", str(args.steps),
                        "--warmup", str(args.warmup), "--gpus", str(args.gpus)] + (["--port"] if args.port else [])
                line = cpu_leg_in_child(argv)
                if "unavailable" in line:
                    line = {"impl": "reference", **line}
                else:
                    line["n_gpus"] = world
                print(json.dumps(line), flush=True)
            return
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
