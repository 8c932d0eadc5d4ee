#!/usr/bin/env python3
"""Batch-1 int4 decode benchmark: tok/s and memory-bandwidth utilisation of the decode megakernel.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config NAME]

One "step" is one decode token of the 3B-class config (40 layers, d 2560, 32 q / 8 kv heads of 80, FFN 8192,
vocab 49160, int4 g128, seeded synthetic weights) after a 128-token prompt; the timed steps are the greedy
decode steps that follow. Rank 0 prints ONE JSON line.

  value         tok/s with the token chain kept on the device (step t+1 reads step t's argmax from HBM),
                CUDA events around the K launches, max over ranks
  e2e           the same metric through the host-facing call: per step the token id goes host->device from pinned
                memory, the kernel runs, the argmax comes back device->host (a sync per token, as chat loops do)
  roofline      HBM: algorithmic bytes per launch (nibbles + bf16 scales + attended K/V rows) / launch time,
                against the measured copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle (OpenMP, all host threads) on a bounded sample of the same workload
  --impl reference  times that CPU implementation alone, same metric and config
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from flint_b200.config import ModelArgs  # noqa: E402
from flint_b200 import packing  # noqa: E402

PROMPT_LEN = 128
HBM_NOMINAL = 8.0e12


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs (read-only queries)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu), "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) > 8 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) > 8 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) > 8:
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_oracle_toks(cfg, packed_cpu, steps: int, pos0: int, warmup: int = 1):
    """Time `steps` decode steps of the CPU oracle (all host threads) at positions pos0.. ; returns tok/s."""
    from oracle import oracle as O
    m = O.OracleModel(cfg, packed_cpu, max_seq=pos0 + steps + 1)
    for _ in range(max(1, warmup)):
        m.decode(1, 0)                               # warm: page the weights in
    tok = 7
    t0 = time.perf_counter()
    for i in range(steps):
        tok = O.argmax_first(m.decode(tok, pos0 + i))
    dt = time.perf_counter() - t0
    return steps / dt, dt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="flint_b200")
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--cpu-steps", type=int, default=100, help="decode steps of the CPU baseline sample (about 10 s of CPU work)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN, help="shorter prompts are for profiler captures only")
    a = ap.parse_args()
    plen = a.prompt_len
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cfg = ModelArgs.from_name(a.config)
    metric, unit = "batch1_int4_decode_tok_per_s", "tok/s"
    workload = (f"{a.config}: batch 1, {plen}-token prompt, greedy decode, int4 g128 sym, "
                f"KV max {cfg.block_size}; weights {cfg.bytes_per_token(0) / 1e9:.2f} GB >> 126 MB L2 (no L2 flush needed)")

    if a.impl == "reference":
        # The reference's CPU-runnable implementation of this path does not exist as compiled code (its kernels are
        # CUDA, its PyTorch int4 op is CUDA-only), so this arm times the oracle port on the host cores.
        if rank != 0:
            return
        torch.manual_seed(0)
        P = packing.synth_packed(cfg, 0, device="cuda" if torch.cuda.is_available() else "cpu")
        Pc = {k: v.cpu() for k, v in P.items()}
        del P
        n = max(1, min(a.steps, 2000))               # one step = one decode token on the host cores (~0.1 s for the 3B model)
        tps, dt = cpu_oracle_toks(cfg, Pc, n, plen, a.warmup)
        cores = os.cpu_count()
        line = {"impl": "reference", "metric": metric, "value": tps, "unit": unit, "n_gpus": a.gpus, "steps": n,
                "warmup": max(1, a.warmup), "ms_per_step": 1000.0 / tps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
                "config": {"workload": workload},
                "cpu_baseline": {"value": tps, "unit": unit, "cores": cores, "kind": "port",
                                 "sample": f"{n} decode steps at positions {plen}.. of the full model"},
                "e2e": {"value": tps, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    from flint_b200.engine import DecodeEngine
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    # N > 1: tensor parallel over the GPUs of the box (strong scaling: the same model, split). The 3B-class model's
    # attention output splits into whole int4 groups only up to 4 ways, so 8 GPUs run two 4-way groups side by side.
    tp = 1
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        tp = world
        while tp > 1 and (cfg.n_local_heads % tp or ((cfg.n_head // tp) * cfg.head_dim) % 128 or
                          (cfg.ffn_padded // 128) % tp or cfg.vocab_size % tp):
            tp //= 2
    n_groups = world // tp
    W = packing.synth_packed(cfg, 0, device=str(dev))
    if tp > 1:
        from flint_b200.tp import make_tp_engine
        groups = [dist.new_group(list(range(g * tp, (g + 1) * tp))) for g in range(n_groups)]
        eng = make_tp_engine(cfg, W, max_seq=cfg.block_size, group=groups[rank // tp], device=dev)
    else:
        eng = DecodeEngine(cfg, W, max_seq=cfg.block_size)
    prompt = torch.randint(0, cfg.vocab_size, (plen,), generator=torch.Generator().manual_seed(1234)).tolist()
    K, Wm = a.steps, max(3, a.warmup)
    if plen + Wm + 2 * K + 4 > cfg.block_size:
        raise SystemExit("steps do not fit the KV cache")

    # ---- prefill token by token (as the reference front-end does, reference: chat.py:85-86), untimed ----
    for pos, t in enumerate(prompt[:-1]):
        eng.decode(t, pos, want_logits=False)
    ring = torch.zeros(K + Wm + 1, dtype=torch.int32, device=dev)
    ring[0] = prompt[-1]
    pos = plen - 1
    for i in range(Wm):                                   # warm-up steps (chained on the device)
        eng.decode_chained(ring[i:i + 1], pos, ring[i + 1:i + 2])
        pos += 1
    eng.check()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- timed region 1: K chained steps, inputs resident in HBM ----
    ring[0] = ring[Wm]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pos0 = pos
    e0.record()
    for i in range(K):
        eng.decode_chained(ring[i:i + 1], pos, ring[i + 1:i + 2])
        pos += 1
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    eng.check()

    # ---- timed region 2: end to end through the host-facing call (pinned H2D token, D2H argmax, per step) ----
    pin_in = torch.zeros(1, dtype=torch.int32).pin_memory()
    pin_out = torch.zeros(1, dtype=torch.int32).pin_memory()
    tok_dev = torch.zeros(1, dtype=torch.int32, device=dev)
    nxt_dev = torch.zeros(1, dtype=torch.int32, device=dev)
    pin_in[0] = int(ring[K].item())
    barrier()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(K):
        tok_dev.copy_(pin_in, non_blocking=True)
        eng.decode_chained(tok_dev, pos, nxt_dev)
        pin_out.copy_(nxt_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        pin_in[0] = int(pin_out[0])
        pos += 1
    e3.record()
    barrier()
    ms_e2e = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3 * 0.0)
    eng.check()

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    n_rep = n_groups                                        # whole-job tokens = (independent TP groups) x K
    tps = n_rep * K / (ms / 1e3)
    tps_e2e = n_rep * K / (ms_e2e / 1e3)
    mean_T = pos0 + (K + 1) / 2.0
    bytes_tok = cfg.bytes_per_token(mean_T) / tp            # algorithmic bytes ONE GPU streams per launch
    weights_only = cfg.bytes_per_token(0) / tp
    peak, which = peaks()
    per_launch_s = (ms / 1e3) / K
    achieved = bytes_tok / per_launch_s / 1e9
    line = {
        "metric": metric, "value": tps, "unit": unit, "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak" if tp == 1 else "strong", "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": workload, "parallelism": "single GPU" if world == 1 else (f"tp{tp}" + (f" x {n_groups} replicas" if n_groups > 1 else "") +
                                                                  ", in-kernel NVLink partial-sum exchange"),
                   "mean_cached_len": mean_T, "bytes_per_token": bytes_tok},
        "mbu_vs_8TBs": bytes_tok * (tps / n_rep) / HBM_NOMINAL,
        "mbu_weights_only_vs_8TBs": weights_only * (tps / n_rep) / HBM_NOMINAL,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": bytes_tok * 1.010, "traffic_note": "ncu: DRAM read+write / algorithmic = 1.010 on one "
                     "launch of this kernel and model (profiles/decode_mega2_granite3b.md), scaled to this run's bytes",
                     "peak_source": which, "kernel": "decode_mega2 (one launch per token)"},
        "e2e": {"value": tps_e2e, "unit": unit, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": K, "clocks": clocks,
    }
    if not a.no_cpu:
        Pc = {k: v.cpu() for k, v in W.items()}
        ctps, cdt = cpu_oracle_toks(cfg, Pc, a.cpu_steps, plen)
        line["cpu_baseline"] = {"value": ctps, "unit": unit, "cores": os.cpu_count(), "kind": "port",
                                "sample": f"{a.cpu_steps} decode steps at positions {plen}.. of the full model "
                                          f"({cdt:.1f} s of CPU work)"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
