#!/usr/bin/env python3
"""Batch-1 int4 decode benchmark: tok/s and memory-bandwidth utilisation of the decode megakernel.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config NAME]

One "step" is one decode token of the 3B-class config (40 layers, d 2560, 32 q / 8 kv heads of 80, FFN 8192,
vocab 49160, int4 g128, seeded synthetic weights) after a 128-token prompt; the timed steps are the greedy
decode steps that follow. Rank 0 prints ONE JSON line.

  value         tok/s of ONE batch-1 stream with the token chain kept on the device (step t+1 reads step t's argmax
                from HBM), CUDA events around the K launches, max over ranks. With N GPUs the model is split N ways
                (tensor parallel, strong scaling); where a model cannot be split N ways, the largest split that
                divides N runs as independent replicas and `config.replicas` says how many (value stays per stream)
  e2e           the same metric through the host-facing call: per step the token id goes host->device from pinned
                memory, the kernel runs, the argmax comes back device->host (a sync per token, as chat loops do)
  roofline      HBM: algorithmic bytes per launch (nibbles + bf16 scales + attended K/V rows) / launch time,
                against the measured copy bandwidth in MEASURED_PEAKS.json
  cpu_baseline  (N = 1 only) the CPU oracle (OpenMP, all host threads) on a bounded sample of the same workload
  long_context, verify_ms, ref_kernel_same_box   (N = 1 only) the other configurations of the path, a few launches each
  tp_check      (N > 1) the tensor-parallel engine against a single-GPU engine on rank 0: first steps' tokens and logits
  --impl reference  times the CPU implementation alone, same metric and config
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
# DRAM read+write bytes / algorithmic bytes of one decode launch, from one ncu capture of this kernel on this model
# (dram__bytes_read.sum + dram__bytes_write.sum = 1.7193 GB against 1.7031 GB algorithmic)
TRAFFIC_RATIO_NCU = 1.010


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
                                          "-i", str(self.gpu), "-lms", "50"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            time.sleep(0.3)                      # the first sample takes a while to arrive
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
    """Time `steps` decode steps of the CPU oracle at positions pos0.. on every host thread; returns (tok/s, s, threads).
    The thread count is set here: launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to their children."""
    from oracle import oracle as O
    threads = O.set_threads(os.cpu_count() or 1)
    m = O.OracleModel(cfg, packed_cpu, max_seq=pos0 + steps + 1)
    for _ in range(max(1, warmup)):
        m.decode(1, 0)                               # warm: page the weights in
    tok = 7
    t0 = time.perf_counter()
    for i in range(steps):
        tok = O.argmax_first(m.decode(tok, pos0 + i))
    dt = time.perf_counter() - t0
    return steps / dt, dt, threads


def timed_chain(eng, ring, pos, n, dev):
    """n chained decode steps from ring[0] at positions pos.. ; CUDA-event milliseconds."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    e0.record()
    for i in range(n):
        eng.decode_chained(ring[i:i + 1], pos + i, ring[i + 1:i + 2])
    e1.record()
    torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1)


def leg_long_context(cfg, eng, dev, cached=32768, steps=12):
    """Long-context configuration: the same engine on a cache pre-filled to 32 768 positions (seeded N(0,1) K/V)."""
    shape = (cfg.n_layer, cached + steps + 8, cfg.n_local_heads, cfg.head_dim)
    g = torch.Generator(device=dev).manual_seed(7)
    kc = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    vc = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    old = (eng.kc, eng.vc)
    eng.bind_kv(kc, vc)
    ring = torch.zeros(steps + 5, dtype=torch.int32, device=dev)
    ring[0] = 17
    timed_chain(eng, ring, cached, 3, dev)
    ring[0] = ring[3]
    ms = timed_chain(eng, ring, cached + 3, steps, dev)
    eng.check()
    eng.bind_kv(*old)
    per = ms / steps
    by = cfg.bytes_per_token(cached + 3 + (steps + 1) / 2.0)
    return {"cached_positions": cached, "steps": steps, "tok_s": 1e3 / per, "ms_per_token": per,
            "achieved_GBs": by / (per / 1e3) / 1e9, "bytes_per_token": by}


def leg_verify(cfg, eng, dev, cache=1024, iters=3):
    """Tree-verify configuration: static trees of 8 / 16 / 26 / 64 nodes over a 1024-token cache; ms per verify pass
    (eager launches; one tree size per GEMM implementation the library chooses from)."""
    from flint_b200.tree import static_tree, tree_mask
    shape = (cfg.n_layer, cache + 128, cfg.n_local_heads, cfg.head_dim)
    g = torch.Generator(device=dev).manual_seed(7)
    kc = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    vc = torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(generator=g)
    old = (eng.kc, eng.vc)
    eng.bind_kv(kc, vc)
    out = {"cache": cache}
    for M in (8, 16, 26, 64):
        parent, depth = static_tree(M)
        am = torch.from_numpy(tree_mask(parent)).to(dev)
        dp = torch.tensor(depth, dtype=torch.int32, device=dev)
        toks = torch.randint(0, cfg.vocab_size, (M,), device=dev, dtype=torch.int32)
        eng.verify(toks, cache, dp, am)
        best = 1e9
        for _ in range(iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize(dev)
            e0.record()
            eng.verify(toks, cache, dp, am)
            e1.record()
            torch.cuda.synchronize(dev)
            best = min(best, e0.elapsed_time(e1))
        eng.check()
        out[str(M)] = best
    eng.bind_kv(*old)
    return out


def leg_ref_kernel(dev, steps=6):
    """The reference's own decode megakernel (built into oracle/_ref from the reference checkout, when it was present at
    build time) and this library, same box, at the only shape the reference kernel supports (40 q / 8 kv heads of 64,
    vocab 100352): tok/s and weights-only MBU against 8 TB/s for both."""
    from oracle import build_ref
    from flint_b200.engine import DecodeEngine
    ref = build_ref.load_module("flint_ref_decode")
    if ref is None:
        return {"unavailable": "oracle/_ref/flint_ref_decode.so was not built"}
    cfg = ModelArgs.from_name("granite-4.1-3b")
    W = packing.synth_packed(cfg, 0, device=str(dev))
    max_seq = 64
    kc = torch.zeros(cfg.n_layer, max_seq, cfg.n_local_heads, cfg.head_dim, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)

    def ref_step(tok, pos):
        h = (W["embed"][tok].float() * cfg.embedding_multiplier).to(torch.bfloat16)
        return ref.decode_mega_launch(W["qkv_q"], W["qkv_s"], W["o_q"], W["o_s"], W["n1"], W["gu_q"], W["gu_s"], W["d_q"],
                                      W["d_s"], W["n2"], W["nf"], W["lm_q"], W["lm_s"], h, kc, vc, pos, cfg.attn_scale,
                                      float(cfg.rope_base), cfg.residual_multiplier, cfg.logits_scaling)
    for p in range(3):
        ref_step(5 + p, p)
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for p in range(steps):
        ref_step(9 + p, 3 + p)
    torch.cuda.synchronize(dev)
    ref_ms = (time.perf_counter() - t0) * 1e3 / steps
    eng = DecodeEngine(cfg, W, max_seq=max_seq)
    ring = torch.zeros(steps + 5, dtype=torch.int32, device=dev)
    ring[0] = 5
    timed_chain(eng, ring, 0, 3, dev)
    ring[0] = ring[3]
    ours_ms = timed_chain(eng, ring, 3, steps, dev) / steps
    eng.check()
    eng.close()
    by = cfg.bytes_per_token(0)
    return {"shape": "granite-4.1-3b (40 q / 8 kv heads of 64, vocab 100352)", "steps": steps,
            "reference": {"tok_s": 1e3 / ref_ms, "mbu_vs_8TBs": by / (ref_ms / 1e3) / HBM_NOMINAL},
            "this_library": {"tok_s": 1e3 / ours_ms, "mbu_vs_8TBs": by / (ours_ms / 1e3) / HBM_NOMINAL}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="flint_b200")
    ap.add_argument("--config", default="granite-3b-class")
    ap.add_argument("--cpu-steps", type=int, default=100, help="decode steps of the CPU baseline sample (about 10 s of CPU work)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the long-context / verify / reference-kernel legs")
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
        tps, dt, threads = cpu_oracle_toks(cfg, Pc, n, plen, a.warmup)
        line = {"impl": "reference", "metric": metric, "value": tps, "unit": unit, "n_gpus": a.gpus, "steps": n,
                "warmup": max(1, a.warmup), "ms_per_step": 1000.0 / tps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
                "config": {"workload": workload},
                "cpu_baseline": {"value": tps, "unit": unit, "cores": threads, "kind": "port",
                                 "sample": f"{n} decode steps at positions {plen}.. of the full model"},
                "e2e": {"value": tps, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    from flint_b200.engine import DecodeEngine
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    # N > 1: tensor parallel over the GPUs of the box (strong scaling: the same model, split).
    tp = 1
    if world > 1:
        import torch.distributed as dist
        from flint_b200.tp import max_tp
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        tp = max_tp(cfg, world)
    n_groups = world // tp
    W = packing.synth_packed(cfg, 0, device=str(dev))
    tp_check = None
    if tp > 1:
        from flint_b200.tp import make_tp_engine
        groups = [dist.new_group(list(range(g * tp, (g + 1) * tp))) for g in range(n_groups)]
        grp = groups[rank // tp]
        eng = make_tp_engine(cfg, W, max_seq=cfg.block_size, group=grp, device=dev)
        # ---- the split engine against a single-GPU engine on the same weights (first group, checked on rank 0) ----
        nchk, vl = 12, cfg.vocab_size // tp
        toks = torch.zeros(nchk + 1, dtype=torch.int32, device=dev)
        toks[0] = 17
        lg = torch.zeros(nchk, cfg.vocab_size, dtype=torch.float32, device=dev)
        for i in range(nchk):
            eng.decode_chained(toks[i:i + 1], i, toks[i + 1:i + 2], lg[i])
        eng.check()
        if rank < tp:
            mine = lg[:, (rank % tp) * vl:(rank % tp + 1) * vl].contiguous()
            parts = [torch.empty_like(mine) for _ in range(tp)] if rank == 0 else None
            dist.gather(mine, parts, dst=0, group=grp)
            if rank == 0:
                full = torch.cat(parts, dim=1)
                one = DecodeEngine(cfg, W, max_seq=64)
                ref = torch.stack([one.decode(int(toks[i]), i).clone() for i in range(nchk)])
                one.check()
                one.close()
                tp_check = {"steps": nchk, "tokens_equal": bool(torch.equal(full.argmax(-1), ref.argmax(-1))),
                            "rel_l2": float((full - ref).norm() / ref.norm())}
                del one, ref, full
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
    torch.cuda.synchronize(dev)
    wall_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    ms_e2e = max(e2.elapsed_time(e3), wall_ms)           # the host's clock includes the syncs the events bracket
    clocks = sampler.stop() if rank == 0 else None
    eng.check()

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    tps = K / (ms / 1e3)                                    # ONE stream (replicas, if any, each run their own)
    tps_e2e = K / (ms_e2e / 1e3)
    mean_T = pos0 + (K + 1) / 2.0
    bytes_tok = cfg.bytes_per_token(mean_T) / tp            # algorithmic bytes ONE GPU streams per launch
    weights_only = cfg.bytes_per_token(0) / tp
    peak, which = peaks()
    per_launch_s = (ms / 1e3) / K
    achieved = bytes_tok / per_launch_s / 1e9
    par = "single GPU" if world == 1 else f"tp{tp}, in-kernel NVLink partial-sum exchange"
    line = {
        "metric": metric, "value": tps, "unit": unit, "n_gpus": world, "steps": K, "warmup": Wm,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak" if world == 1 else "strong", "vs_baseline": None,
        "dtype": "int4 weights, bf16 activations, fp32 accumulate", "data": "synthetic",
        "config": {"workload": workload, "parallelism": par, "replicas": n_groups,
                   "mean_cached_len": mean_T, "bytes_per_token": bytes_tok},
        "mbu_vs_8TBs": bytes_tok * tps / HBM_NOMINAL,
        "mbu_weights_only_vs_8TBs": weights_only * tps / HBM_NOMINAL,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": bytes_tok * TRAFFIC_RATIO_NCU,
                     "traffic_source": f"not measured in this run: algorithmic bytes x {TRAFFIC_RATIO_NCU} (DRAM read+write / "
                                       "algorithmic of one ncu-captured launch of this kernel on this model)",
                     "peak_source": which, "kernel": "decode_mega2 (one launch per token)"},
        "e2e": {"value": tps_e2e, "unit": unit, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": K, "clocks": clocks,
    }
    if tp_check is not None:
        line["tp_check"] = tp_check
    if world == 1 and not a.no_extra:
        for name, fn in (("long_context", lambda: leg_long_context(cfg, eng, dev)),
                         ("verify_ms", lambda: leg_verify(cfg, eng, dev))):
            try:
                line[name] = fn()
            except Exception as exc:                      # an extra leg must not cost the headline line
                line[name] = {"error": repr(exc)[:200]}
    if world == 1 and not a.no_cpu:
        Pc = {k: v.cpu() for k, v in W.items()}
        ctps, cdt, threads = cpu_oracle_toks(cfg, Pc, a.cpu_steps, plen)
        line["cpu_baseline"] = {"value": ctps, "unit": unit, "cores": threads, "kind": "port",
                                "sample": f"{a.cpu_steps} decode steps at positions {plen}.. of the full model "
                                          f"({cdt:.1f} s of CPU work)"}
        del Pc
    if world == 1 and not a.no_extra:
        eng.close()
        del eng, W
        torch.cuda.empty_cache()
        try:
            line["ref_kernel_same_box"] = leg_ref_kernel(dev)
        except Exception as exc:
            line["ref_kernel_same_box"] = {"error": repr(exc)[:200]}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
