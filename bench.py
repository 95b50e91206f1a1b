#!/usr/bin/env python
"""bench.py - decoded audio frames/s of the Dia-1.6B decode path on B200 (BASELINE.json metric).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1]): Dia-1.6B, bf16 weights, ONE transcript, CFG batch 2, a full
3072-token generation = 3071 autoregressive decode steps.  A bench "step" is one such generation.
With N > 1 GPUs every rank runs its own utterance (replicas, no collective on the data
path); `value` is the sum over ranks divided by the slowest rank's time (weak scaling).

  value  frames/s of the decode loop with everything already resident in HBM (encoder output,
         cross-KV, token grid), timed on the device with CUDA events on the launching stream.
  e2e    frames/s through the public API, `Dia.generate(text, output="codes")` + `.cpu()`: text in host
         memory in, codes in host memory out; encoder, cross-KV precompute, H2D/D2H inside the region.
  roofline     the step kernel: algorithmic bytes of the steps in a launch / event-timed launch duration,
               against the measured HBM copy bandwidth in MEASURED_PEAKS.json.
  cpu_baseline the CPU port of the reference's own algorithm (oracle/, kind "port": the reference is
               Python and cannot travel to the GPU box) timed on this box's host cores.

`--impl reference` times that CPU port alone (rank 0 only).

`--lm` leaves that workload aside and measures the decoder-only language-model path (Pubopel, random weights) at layer
sizes of a real model: prefill and decode throughput through `CausalLM`, and its GEMM / attention kernels beside Dia's
at equal size (one JSON line, metric `lm_layer_throughput`).  `--lm --lm-design luketar` measures the Luketar design
beside Kupelix and Pubopel at equal width and its mixers beside Kupelix's.  `--lm --lm-design fipadra` measures the Fipadra
design beside Luketar at equal width and its mixers beside their likes in Luketar and Kupelix.  `--lm --lm-design kupelix` measures the Kupelix design
instead: its prefill and decode throughput beside Pubopel's at equal width, heads and vocabulary, its attention kernel
beside Pubopel's on the same causal workload, and its recurrence kernels against the bytes and state updates they must move.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

METRIC = "decoded_audio_frames_per_s"
UNIT = "frames/s"
MAX_TOKENS = 3072
WEIGHT_SEED = 5
FRAME_RATE = 44100 / 512          # 86.13 frames per second of audio


VARIANTS = {
    "dense": "Dia-1.6B",
    "mlp-pruned": "Dia-1.6B with mlp.wo structurally pruned along dim 0 (offline_prune.py --prune-dim 0, L2 norm; "
                  "BASELINE.json configs[3] 'reduced MLP width')",
    "2to4": "Dia-1.6B with every dense kernel 2:4-pruned along K (BASELINE.json configs[3], unstructured-sparse variant)",
    "structured": "Dia-1.6B after the stock offline_prune.py call: apply_structured_pruning(model, amount, dim=0, n=2) on "
                  "EVERY DenseGeneral (input rows zeroed; the engine drops them: K-row compaction + reduced MLP width)",
}


def workload_config(text_len: int, world: int, variant: str = "dense", amount: float = 0.0) -> dict:
    """The `config` object both arms print (BASELINE.json configs[1], one utterance per GPU)."""
    model = VARIANTS[variant] + (f", amount {amount}" if variant in ("mlp-pruned", "structured") else "")
    return {"workload": f"{model} bf16 weights, single transcript per GPU, CFG batch 2, full 3072-token "
                        "generation (3071 decode steps), reference default sampling T=1.3 top_p=0.95 top_k=35",
            "precision": "bf16 weights; fp32 activations, accumulation, softmax and KV cache",
            "weights": f"random-init seed {WEIGHT_SEED}, channel-0 EOS column zeroed so no early EOS",
            "l2": "inputs larger than L2: 2.53 GB of weights streamed per decode step",
            "frame": "1 frame = 1 decode step = 9 codes = 512 samples @ 44.1 kHz",
            "text_len": text_len, "parallelism": f"replicas x{world}, no data-path collective"}


def algorithmic_bytes(cfg, slot: int, text_len: int, kv_elem: int = 4, n_hidden: int | None = None,
                      weight_scale: float = 1.0, dense_bytes: int | None = None) -> int:
    """Bytes one decode step must move: bf16 weights of the 18 layers + logits head, fp32 norm weights, 9 embedding rows,
    plus self-KV rows read / appended and the valid cross-KV rows of the conditional row.  Pruned variants:
    ``n_hidden`` = live MLP width of a structurally pruned model; ``weight_scale`` = 0.5625 for 2:4 (half the
    values + 2 bits of metadata per kept value)."""
    d, e = cfg.model.decoder, cfg.model.encoder
    D, F, hd = d.n_embd, n_hidden or d.n_hidden, 128
    nq, nkv, nc = d.gqa_query_heads * hd, d.kv_heads * hd, d.cross_query_heads * hd
    per_layer = D * (nq + 2 * nkv) + nq * D + D * nc + nc * D + D * 2 * F + F * D
    w = int(2 * weight_scale * (d.n_layer * per_layer + D * cfg.data.channels * cfg.model.tgt_vocab_size))
    if dense_bytes is not None:        # row-compacted (structurally pruned) model: the live kernels as the engine streams them
        w = int(dense_bytes)
    w += 4 * (3 * d.n_layer + 1) * D + 4 * cfg.data.channels * D
    kv_row = d.n_layer * 2 * 2 * nkv * kv_elem            # K and V, both CFG rows, all layers, one slot
    cross = d.n_layer * 2 * nc * kv_elem * text_len       # K and V, conditional row only
    return w + kv_row * (slot + 1) + cross


class ClockSampler:
    """nvidia-smi sampled during the timed region (B200_PROFILING.md clocks line)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        load = [x for x in sm if mx and x > 0.5 * mx] or sm
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def measured_peak() -> tuple[float, str]:
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return 6650.0, "fallback (B200_PROFILING.md)"


def build_cpu_model(seed: int, suppress_eos: bool):
    """fp32 CPU DiaModel with the shared synthetic recipe; returns (Dia, state dict clone or None)."""
    import torch
    from dia_tts_prune_b200.config import dia_1_6b_config
    from dia_tts_prune_b200.model import Dia
    from dia_tts_prune_b200 import synthetic as SY
    cfg = dia_1_6b_config()
    dia = Dia(cfg, "float32", torch.device("cpu"))
    SY.init_synthetic_(dia.model.named_parameters(), seed)
    if suppress_eos:
        # random weights would emit EOS on channel 0 within ~1000 steps and end the utterance early;
        # a zero EOS column keeps all 3071 steps running
        with torch.no_grad():
            dia.model.decoder.logits_dense.weight[:, 0, cfg.data.audio_eos_value] = 0.0
    return dia, cfg


def cpu_port_frames_per_s(sd, cfg, text: str, n_steps: int, threads: int, lean_steps: int = 0) -> dict:
    """The oracle port of the reference's decode loop, timed on the host (dead cross-attention K/V
    re-projection kept, as shipped: dia/layers.py:274-275).  ``lean_steps`` > 0 also times the same loop with that
    dead projection skipped (identical outputs; BASELINE.md section 3's "useful-work" CPU figure)."""
    import torch
    from oracle import dia_oracle as O
    torch.set_num_threads(threads)
    t0 = time.perf_counter()
    tr = O.generate(sd, cfg, text, max_tokens=1 + n_steps, temperature=0.0, cfg_scale=3.0, dead_cross_kv=True,
                    time_steps=True)
    total = time.perf_counter() - t0
    loop = sum(tr.step_seconds)
    out = {"value": len(tr.step_seconds) / loop, "unit": UNIT, "cores": threads, "kind": "port",
           "sample": f"{len(tr.step_seconds)} greedy decode steps (cache slots 0..{len(tr.step_seconds) - 1}) of the same "
                     f"Dia-1.6B fp32 workload on the host (CFG batch 2, dead cross-K/V projection kept as shipped), loop "
                     f"{loop:.1f}s; one-time encoder+cross-KV prepare {total - loop:.1f}s excluded"}
    if lean_steps > 0:
        tr = O.generate(sd, cfg, text, max_tokens=1 + lean_steps, temperature=0.0, cfg_scale=3.0, dead_cross_kv=False,
                        time_steps=True)
        out["lean_value"] = len(tr.step_seconds) / sum(tr.step_seconds)
        out["lean_note"] = (f"same loop over {len(tr.step_seconds)} steps with the reference's dead per-step cross-attention "
                            "K/V re-projection skipped (outputs identical)")
    return out


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from dia_tts_prune_b200 import synthetic as SY
    threads = os.cpu_count() or 1
    dia, cfg = build_cpu_model(WEIGHT_SEED, suppress_eos=True)
    sd = {k: v.detach() for k, v in dia.model.named_parameters()}
    eff = dia._effective_text(SY.DEFAULT_TRANSCRIPT, None)                 # speaker tags are one byte each
    text_len = len(eff.encode("utf-8").replace(b"[S1]", b"\x01").replace(b"[S2]", b"\x02"))
    per_step = max(2, args.ref_decode_steps)
    vals, t_all = [], time.perf_counter()
    for i in range(args.warmup + args.steps):
        r = cpu_port_frames_per_s(sd, cfg, SY.DEFAULT_TRANSCRIPT, per_step, threads)
        if i >= args.warmup:
            vals.append(r)
    v = statistics.mean(x["value"] for x in vals)
    line = {"metric": METRIC, "value": v, "unit": UNIT, "impl": "reference", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": 1000.0 * per_step / v, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(text_len, max(1, args.gpus)),
            "note": f"reference arm: the CPU port of the reference's own fp32 loop; every bench step is a bounded sample of "
                    f"{per_step} greedy decode steps of that workload (precision fp32 on the host, not bf16)",
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "sample": vals[-1]["sample"]},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0, "rtfx": v / FRAME_RATE, "wall_s": time.perf_counter() - t_all}
    print(json.dumps(line), flush=True)


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist
    from dia_tts_prune_b200 import synthetic as SY
    from dia_tts_prune_b200.engine import launch_count

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))

    dia, cfg = build_cpu_model(WEIGHT_SEED, suppress_eos=True)
    if args.variant != "dense":
        # BASELINE.json configs[3]: the weight producers of dia/pruning_utils.py (+ the 2:4 mask) on the same model
        import torch.nn.utils.prune as prune
        from dia_tts_prune_b200 import pruning_utils as PU
        if args.variant == "mlp-pruned":
            for layer in dia.model.decoder.layers:
                prune.ln_structured(layer.mlp.wo, "weight", amount=args.prune_amount, n=2, dim=0)
        elif args.variant == "structured":
            PU.apply_structured_pruning(dia.model, args.prune_amount, dim=0, n=2)
            with torch.no_grad():        # keep the zeroed channel-0 EOS column from coming back as the only live one
                dia.model.decoder.logits_dense.weight[:, 0, cfg.data.audio_eos_value] = 0.0
        else:
            PU.apply_2to4_pruning(dia.model.decoder)
        PU.make_pruning_permanent(dia.model)
    sd_cpu = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        sd_cpu = {k: v.detach().clone() for k, v in dia.model.named_parameters()}
    # configs[1]: bf16 weights.  Values are bf16-representable, so this cast is exact.
    SY.cast_dense_kernels_(dia.model, torch.bfloat16)
    dia.compute_dtype = torch.bfloat16
    dia.device = dev
    dia.model.to(dev)
    dia.model.eval()
    text = SY.DEFAULT_TRANSCRIPT          # the same transcript on every rank and at every N: like-for-like weak scaling
    sampling = dict(cfg_scale=3.0, temperature=1.3, top_p=0.95, top_k=35)

    # ---- resident inputs for the device-timed loop --------------------------------------------------
    eff = dia._effective_text(text, None)
    with torch.inference_mode():
        dec_state, dec_out = dia._prepare_generation(eff, None, False)
    pristine = dec_out.generated_tokens.clone()
    text_len = dec_state.text_len
    eng_width = dia.model.decoder.engine().n_hidden           # < n_hidden when dead MLP neurons were dropped
    w_scale = 0.5625 if args.variant == "2to4" else 1.0
    live_bytes = dia.model.decoder.engine().weight_stream_bytes if args.variant == "structured" else None

    def one_generation(profile=None) -> int:
        for c in dec_state.self_attn_cache:
            c.current_idx = 0
        with torch.inference_mode():
            dec_out.generated_tokens.copy_(pristine)
            last = dia._run_loop(dec_state, dec_out, MAX_TOKENS, sampling["cfg_scale"], sampling["temperature"],
                                 sampling["top_p"], sampling["top_k"], 1234, False, profile=profile)
        return last + 1 - (dec_out.prefill_step - 1)        # loop iterations executed (the loop ends by `break`)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        one_generation()
    sampler = ClockSampler(local)
    sync_all()
    sampler.start()
    launches0 = launch_count()
    profile: list = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps_run = 0
    for _ in range(args.steps):
        steps_run += one_generation(profile)
    e1.record()
    sync_all()
    launches = launch_count() - launches0
    dev_ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    frames_dev = steps_run                                     # one decode step = one frame (9 codes)

    # roofline of the step kernel: per-launch algorithmic bytes / event-timed duration
    k_bytes = k_ms = 0.0
    for (a, b, slot0, n) in profile:
        k_ms += a.elapsed_time(b)
        k_bytes += sum(algorithmic_bytes(cfg, slot0 + i, text_len, n_hidden=eng_width, weight_scale=w_scale, dense_bytes=live_bytes)
                       for i in range(n))
    peak, peak_src = measured_peak()
    achieved = k_bytes / (k_ms * 1e-3) / 1e9

    # ---- end to end through the public API, host buffers in and out ---------------------------------------
    def one_e2e():
        codes = dia.generate(text, max_tokens=MAX_TOKENS, seed=1234, output="codes", **{
            "cfg_scale": sampling["cfg_scale"], "temperature": sampling["temperature"], "top_p": sampling["top_p"],
            "cfg_filter_top_k": sampling["top_k"]})
        host = codes.cpu()
        return dia.last_stats["steps"], host
    for _ in range(min(args.warmup, 2)):
        one_e2e()
    sync_all()
    t0 = time.perf_counter()
    e2e_steps, d2h = 0, 0
    for _ in range(args.steps):
        n, host = one_e2e()
        e2e_steps += n
        d2h = host.numel() * host.element_size()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        dist.barrier()
    h2d = 2 * cfg.data.text_length * 8 + 4                     # [2, text_length] int64 text tokens (+ seed)

    # ---- reduce over ranks: max time, sum frames ------------------------------------------------------------
    t = torch.tensor([dev_ms, e2e_s, float(frames_dev), float(e2e_steps), k_ms, k_bytes, float(launches)],
                     dtype=torch.float64, device=dev)
    per_rank_ms = [dev_ms / args.steps]
    if world > 1:
        tmax, tsum = t.clone(), t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
        every = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(every, t)
        per_rank_ms = [x[0].item() / args.steps for x in every]
        dev_ms, e2e_s = tmax[0].item(), tmax[1].item()
        frames_dev, e2e_steps, launches = tsum[2].item(), tsum[3].item(), tsum[6].item()
        k_ms, k_bytes = tsum[4].item() / world, tsum[5].item() / world            # roofline: mean over the replicas
        achieved = k_bytes / (k_ms * 1e-3) / 1e9
    value = frames_dev / (dev_ms * 1e-3)
    e2e_value = e2e_steps / e2e_s

    # ---- BASELINE.json configs[4] as a second field of the same line: 64 transcripts sharded over the ranks --------------------
    batch_field = None
    if args.batch_utterances > 0 and args.variant == "dense":
        from dia_tts_prune_b200 import replicas
        texts = replicas.shard([SY.synthetic_transcript(i) for i in range(args.batch_utterances)], world, rank)
        if texts:
            dia.generate_batch(texts[: args.per_launch], max_tokens=64, seed=1, max_utterances=args.per_launch)   # warm-up: repack
        sync_all()
        r = batch_workload(dia, cfg, texts, MAX_TOKENS, args.per_launch, dev) if texts else {"frames": 0, "secs": 0.0}
        frames_b, secs_b = replicas.reduce_throughput(r["frames"], r["secs"], device=dev)
        if rank == 0 and secs_b > 0:
            vb = frames_b / secs_b
            batch_field = {"workload": f"BASELINE configs[4]: {args.batch_utterances} synthetic transcripts (60-200 bytes) x "
                                       f"{MAX_TOKENS} tokens sharded round-robin over {world} GPU(s), {args.per_launch} "
                                       "utterances per kernel launch, end to end through Dia.generate_batch",
                           "value": vb, "unit": UNIT, "scaling": "strong", "frames": frames_b, "wall_s": secs_b,
                           "per_gpu_frames_per_s": vb / world, "n_per_launch": r.get("n_per_launch"),
                           "roofline_frames_per_s_per_gpu": r.get("roofline_frames_per_s_per_gpu"),
                           "frac_of_roofline": vb / world / r["roofline_frames_per_s_per_gpu"]
                           if r.get("roofline_frames_per_s_per_gpu") else None,
                           "rtfx": vb / FRAME_RATE}

    cpu_base = None
    if sd_cpu is not None:
        cpu_base = cpu_port_frames_per_s(sd_cpu, cfg, SY.DEFAULT_TRANSCRIPT, args.cpu_decode_steps, os.cpu_count() or 1,
                                         lean_steps=args.cpu_decode_steps)

    if rank == 0:
        # DRAM bytes per launch from the committed `ncu --set full` capture (per decode STEP there, scaled to the mean
        # number of steps of the launches timed here, so that it compares with algorithmic_bytes_per_launch)
        traffic, traffic_src = None, None
        steps_per_launch = frames_dev / world / max(1, len(profile))
        try:
            with open(os.path.join(REPO, "profiles", "step_kernel_traffic.json")) as f:
                tj = json.load(f)
            if args.variant == "dense":
                traffic = tj["dram_bytes_per_step"] * steps_per_launch
                traffic_src = tj.get("source")
        except Exception:
            pass
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": dict(workload_config(text_len, world, args.variant, args.prune_amount),
                           **({"engine_mlp_width": eng_width} if args.variant != "dense" else {})),
            "decode_ms_per_frame": dev_ms / (frames_dev / world),
            "rtfx": value / world / FRAME_RATE,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1000.0 * e2e_s / args.steps},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_src, "kernel": "dia_step_kernel",
                         "launches_timed": len(profile), "steps_per_launch": steps_per_launch,
                         "traffic_source": traffic_src,
                         "algorithmic_bytes_per_launch": k_bytes / max(1, len(profile)),
                         "algorithmic_bytes_per_step": k_bytes / max(1.0, frames_dev / world)},
            "per_rank_ms_per_step": per_rank_ms,
            "cpu_baseline": cpu_base,
            "clocks": clocks,
            "batch": batch_field,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def batch_workload(dia, cfg, texts, max_tokens: int, per_launch: int, dev) -> dict:
    """BASELINE.json configs[4] on ONE rank: its share of the transcripts through ``Dia.generate_batch`` (``per_launch``
    utterances per kernel launch: 2N rows share one pass over the weights), host text in, host codes out.  Returns frames,
    wall seconds and the roofline of this shape (bytes = W + N * 36 864 * e * (t + 2 Lt) per step of N
    frames)."""
    import torch
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    outs = dia.generate_batch(texts, max_tokens=max_tokens, seed=1234, max_utterances=per_launch)
    host = [o.cpu() for o in outs]
    torch.cuda.synchronize(dev)
    secs = time.perf_counter() - t0
    st = dia.last_stats
    frames = st["steps"]
    # roofline at this N: the mean context of a full generation, the mean text length of the transcripts
    lt = sum(len(dia._effective_text(t, None).encode("utf-8").replace(b"[S1]", b"\x01").replace(b"[S2]", b"\x02"))
             for t in texts) / max(1, len(texts))
    n = min(per_launch, len(texts))
    w_bytes = algorithmic_bytes(cfg, 0, 0) - cfg.model.decoder.n_layer * 2 * 2 * cfg.model.decoder.kv_heads * 128 * 4
    kv_per_utt = algorithmic_bytes(cfg, max_tokens // 2, int(lt)) - w_bytes
    peak, _ = measured_peak()
    roof = n / ((w_bytes + n * kv_per_utt) / (peak * 1e9))            # frames/s per GPU at the copy peak
    return {"frames": frames, "secs": secs, "loop_s": st["loop_s"], "prepare_s": st["prepare_s"], "n_per_launch": n,
            "roofline_frames_per_s_per_gpu": roof, "d2h_bytes": sum(h.numel() * h.element_size() for h in host)}


def run_batch(args) -> None:
    """BASELINE.json configs[4]: `--utterances M` synthetic transcripts sharded round-robin over the ranks (replicas, no
    data-path collective); every rank decodes its share `--per-launch` utterances at a time in one kernel.  Prints one
    JSON line with the whole-job throughput (sum of frames over ranks / slowest rank's wall time).  Not the headline
    line: the driver's `python bench.py` (no --utterances) stays configs[1] and carries this as its "batch" field."""
    import torch
    import torch.distributed as dist
    from dia_tts_prune_b200 import replicas, synthetic as SY

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dia, cfg = build_cpu_model(WEIGHT_SEED, suppress_eos=True)
    SY.cast_dense_kernels_(dia.model, torch.bfloat16)
    dia.compute_dtype = torch.bfloat16
    dia.device = dev
    dia.model.to(dev)
    dia.model.eval()
    texts = [SY.synthetic_transcript(i) for i in range(args.utterances)]
    mine = replicas.shard(texts, world, rank)
    dia.generate_batch(mine[: args.per_launch], max_tokens=min(args.max_tokens, 64), seed=1, max_utterances=args.per_launch)
    if world > 1:
        dist.barrier()
    r = batch_workload(dia, cfg, mine, args.max_tokens, args.per_launch, dev)
    frames_all, secs_max = replicas.reduce_throughput(r["frames"], r["secs"], device=dev)
    if rank == 0:
        value = frames_all / secs_max
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "higher_is_better": True,
            "scaling": "strong", "data": "synthetic", "dtype": "bf16",
            "config": {"workload": f"{args.utterances} independent synthetic transcripts (60-200 bytes) sharded round-robin "
                                   f"over {world} GPU(s), {args.per_launch} utterances per kernel launch, max_tokens "
                                   f"{args.max_tokens} each, CFG batch 2 per utterance, default sampling; end to end "
                                   "through Dia.generate_batch (host text in, host codes out)",
                       "parallelism": f"replicas x{world}, no data-path collective"},
            "frames": frames_all, "wall_s": secs_max, "rtfx": value / FRAME_RATE,
            "per_gpu_frames_per_s": value / world,
            "roofline_frames_per_s_per_gpu": r["roofline_frames_per_s_per_gpu"],
            "frac_of_roofline": value / world / r["roofline_frames_per_s_per_gpu"]}), flush=True)
    if world > 1:
        dist.destroy_process_group()



# ---- --lm: the decoder-only language-model path at layer sizes of a real model, beside Dia's kernels at equal size ------
LM_SIZES = {
    # width 2048, 16 x 128 query heads over 4 key/value heads: the shape of Dia-1.6B's decoder self-attention; two routed
    # experts of 2048 + a shared one of 4096 = 8192 active hidden units per token, the width of Dia's decoder MLP
    "w2048": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=128, experts=8, top=2, expert_ff=2048, shared_ff=4096,
                  vocab=32768, window=1024, keep_first=4),
    "w1024": dict(width=1024, layers=4, heads=8, kv_heads=2, dim=128, experts=16, top=2, expert_ff=512, shared_ff=1024,
                  vocab=16384, window=512, keep_first=4),
}


def _event_ms(fn, warmup: int, steps: int, flush=None) -> float:
    """Median CUDA-event time of fn() on the current stream; `flush` (a buffer larger than L2) is rewritten in between."""
    import torch
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(steps):
        if flush is not None:
            flush.add_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def run_lm(args) -> None:
    import torch
    from dia_tts_prune_b200 import engine as DE
    from dia_tts_prune_b200 import synthetic as SY
    from dia_tts_prune_b200.lm_config import PubopelConfig
    from dia_tts_prune_b200.lm_engine import launch_count, linear
    from dia_tts_prune_b200.lm_model import CausalLM

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        hbm, tf, src = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), "measured"
    except Exception:
        hbm, tf, src = 6650.0, 1590.0, "fallback"
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)             # > the 126 MB L2
    W, K = max(args.warmup, 3), max(args.steps, 3)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = launch_count()
    out = {}
    for name in (args.lm_sizes.split(",") if args.lm_sizes else LM_SIZES):
        sz = LM_SIZES[name]
        cfg = SY.pubopel_config(**sz)
        weights = SY.pubopel_weights(cfg, WEIGHT_SEED, dev)
        T, ctx = args.lm_prompt, args.lm_context
        model = CausalLM(PubopelConfig.model_validate(cfg), weights, dtype="bfloat16", device=dev,
                         max_tokens=max(T, 8 * (ctx + 32 * (K + 2))) + 64, max_sequences=8, page_size=64, max_rows=args.lm_rows)
        del weights
        D, H, G, d = sz["width"], sz["heads"], sz["kv_heads"], sz["dim"]
        nq, nk, F, Sf, E, top, V, L = H * d, G * d, sz["expert_ff"], sz["shared_ff"], sz["experts"], sz["top"], sz["vocab"], sz["layers"]
        win, keep = sz["window"], sz["keep_first"]
        g = torch.Generator().manual_seed(7)
        toks = torch.randint(0, V, (T,), generator=g).tolist()
        res = {"config": sz}

        # -- prefill: one prompt of T tokens through the step function (portions of --lm-rows rows), logits of the last token
        def prefill():
            model.run_step([{"id": "p", "tokens": toks, "want": [T - 1]}], ["p"])
        ms = _event_ms(prefill, W, K, flush)
        seen = sum(min(i + 1, win) + min(keep, max(0, i + 1 - win)) for i in range(T))
        flops = L * (2.0 * T * D * (nq + nk) + 2.0 * T * nq * D + 2.0 * T * D * E + top * 6.0 * T * D * F + 6.0 * T * D * Sf
                     + 4.0 * d * H * seen) + 2.0 * D * V
        res["prefill"] = {"tokens": T, "rows_per_step": args.lm_rows, "ms": ms, "tokens_per_s": T / ms * 1e3, "model_tflops": flops / ms / 1e9,
                          "frac_of_bf16_peak": flops / ms / 1e9 / tf}

        # -- decode: B sequences of `ctx` tokens each, one token per sequence per step, teacher-forced, device-timed
        for B in (1, 8):
            for b in range(B):
                model.run_step([{"id": f"d{b}", "tokens": toks[:ctx], "want": []}])
            n_dec = 32
            def decode():
                for t in range(n_dec):
                    model.run_step([{"id": f"d{b}", "tokens": [toks[(ctx + t) % T]], "want": [0]} for b in range(B)])
            ms = _event_ms(decode, 1, K) / n_dec
            for b in range(B):
                model.state.close(f"d{b}")
            entry = {"context": ctx, "ms_per_step": ms, "tokens_per_s": B / ms * 1e3}
            if B == 1:      # bytes one step must read: this token's share of the weights (bf16) and its visible keys + values (fp32)
                n_keys = min(ctx, win) + min(keep, max(0, ctx - win))
                byt = L * (2.0 * (D * (nq + nk) + nq * D + E * D + top * 3 * D * F + 3 * D * Sf) + 8.0 * n_keys * G * d) + 2.0 * D * V
                entry.update(algorithmic_bytes=byt, gb_per_s=byt / ms / 1e6, frac_of_hbm_peak=byt / ms / 1e6 / hbm)
            res[f"decode_b{B}"] = entry

        # -- end to end: generate() through the scheduler, prompts from host lists, sampled ids back on the host
        prompts = [toks[:256] for _ in range(8)]
        model.generate(prompts[:1], max_new_tokens=4)
        t0 = time.perf_counter()
        outs = model.generate(prompts, max_new_tokens=64)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        res["generate_e2e"] = {"requests": 8, "prompt": 256, "new_tokens": 64, "wall_s": wall,
                               "new_tokens_per_s": sum(len(o) for o in outs) / wall}

        # -- kernels alone, beside Dia's at equal size
        M = min(args.lm_rows, T)
        kern = {}
        for label, (N_, K_) in {"qk_proj": (nq + nk, D), "o_proj": (D, nq), "shared_gate_up": (2 * Sf, D)}.items():
            a = torch.randn(M, K_, device=dev)
            w = (torch.randn(N_, K_, device=dev) * K_ ** -0.5).to(torch.bfloat16)
            ms_lm = _event_ms(lambda: linear(a, w, tensor_cores=True), W, K, flush)
            kern[label] = {"M": M, "N": N_, "K": K_, "pubopel_ms": ms_lm, "pubopel_frac_of_bf16_peak": 2.0 * M * N_ * K_ / ms_lm / 1e9 / tf}
            if DE.dense_supported(M, N_, K_):
                ms_dia = _event_ms(lambda: DE.dense_forward(a, w), W, K, flush)
                kern[label].update(dia_ms=ms_dia, dia_frac_of_bf16_peak=2.0 * M * N_ * K_ / ms_dia / 1e9 / tf)
        # attention: T rows of one sequence, full causal (no window) so that both kernels do the same work
        eng = model.engine
        full = CausalLM(PubopelConfig.model_validate(SY.pubopel_config(**{**sz, "layers": 1, "window": None, "vocab": 256,
                                                                           "experts": 1, "top": 1, "expert_ff": 8, "shared_ff": None})),
                        SY.pubopel_weights(SY.pubopel_config(**{**sz, "layers": 1, "window": None, "vocab": 256, "experts": 1,
                                                                "top": 1, "expert_ff": 8, "shared_ff": None}), 3, dev),
                        dtype="float32", device=dev, max_tokens=T + 64, max_sequences=2, page_size=64, max_rows=args.lm_rows)
        qk = torch.randn(T, nq + nk, device=dev)
        def lm_attn():
            seq = full.state.open("a")
            for r0 in range(0, T, args.lm_rows):
                n = min(args.lm_rows, T - r0)
                full.state.reserve(seq, n)
                full.engine.op_attention(0, qk[r0:r0 + n], [(seq, n, r0)])
                full.state.advance(seq, n)
            full.state.close("a")
        ms_lm = _event_ms(lm_attn, 2, K, flush)
        a_flops = 4.0 * d * H * T * (T + 1) / 2
        kern["attention_causal"] = {"T": T, "heads": H, "kv_heads": G, "dim": d, "pubopel_ms": ms_lm,
                                    "pubopel_tflops_fp32": a_flops / ms_lm / 1e9}
        if d == 128:
            q4 = torch.randn(1, T, H, d, device=dev)
            kc, vc = torch.randn(1, G, T, d, device=dev), torch.randn(1, G, T, d, device=dev)
            ms_dia = _event_ms(lambda: DE.attention_rows(q4, kc, vc, T, 0, [T]), 2, K, flush)
            kern["attention_causal"].update(dia_ms=ms_dia, dia_tflops_fp32=a_flops / ms_dia / 1e9)
        res["kernels"] = kern
        out[name] = res
        model.engine.close(); full.engine.close()
        del model, full
        torch.cuda.empty_cache()
    clocks = sampler.stop()
    print(json.dumps({"metric": "lm_layer_throughput", "impl": "ours", "n_gpus": 1, "steps": K, "warmup": W, "dtype": "bf16",
                      "data": "synthetic (random weights, random token ids)", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
                      "timing": "CUDA events, median; a 160 MB buffer is rewritten between timed iterations (L2 flush)",
                      "gpu_launches": launch_count() - launches0, "clocks": clocks, "lm": out}))


# ---- --lm --lm-design kupelix: the Kupelix design beside Pubopel at equal width, and its kernels beside Pubopel's ---------
KUPELIX_SIZES = {
    # the widths, head shapes and vocabularies of LM_SIZES; a dense feed-forward as wide as Pubopel's active hidden units
    "w2048": dict(width=2048, kinds=["attention", "hgrn2", "channel_delta", "attention"], heads=16, kv_heads=4, dim=128, vdim=128,
                  ff=8192, vocab=32768),
    "w1024": dict(width=1024, kinds=["attention", "hgrn2", "channel_delta", "attention"], heads=8, kv_heads=2, dim=128, vdim=128,
                  ff=2048, vocab=16384),
}


def _lm_prefill_decode(model, toks, T, ctx, W, K, flush) -> dict:
    """Prefill of one T-token prompt and teacher-forced decoding of 1 and 8 sequences at `ctx` tokens, device-timed."""
    def prefill():
        model.run_step([{"id": "p", "tokens": toks, "want": [T - 1]}], ["p"])
    ms = _event_ms(prefill, W, K, flush)
    res = {"prefill": {"tokens": T, "ms": ms, "tokens_per_s": T / ms * 1e3}}
    for B in (1, 8):
        for b in range(B):
            model.run_step([{"id": f"d{b}", "tokens": toks[:ctx], "want": []}])
        n_dec = 32
        def decode():
            for t in range(n_dec):
                model.run_step([{"id": f"d{b}", "tokens": [toks[(ctx + t) % T]], "want": [0]} for b in range(B)])
        ms = _event_ms(decode, 1, K) / n_dec
        for b in range(B):
            model.state.close(f"d{b}")
        res[f"decode_b{B}"] = {"context": ctx, "ms_per_step": ms, "tokens_per_s": B / ms * 1e3}
    return res


def run_lm_kupelix(args) -> None:
    import torch
    from dia_tts_prune_b200 import synthetic as SY
    from dia_tts_prune_b200.lm_config import KupelixConfig, PubopelConfig
    from dia_tts_prune_b200.lm_engine import launch_count
    from dia_tts_prune_b200.lm_model import CausalLM

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        hbm, tf, src = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), "measured"
    except Exception:
        hbm, tf, src = 6650.0, 1590.0, "fallback"
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)             # > the 126 MB L2
    W, K = max(args.warmup, 3), max(args.steps, 3)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = launch_count()
    out = {}
    T, ctx, R = args.lm_prompt, args.lm_context, args.lm_rows
    for name in (args.lm_sizes.split(",") if args.lm_sizes else KUPELIX_SIZES):
        sz, psz = KUPELIX_SIZES[name], LM_SIZES[name]
        D, H, G, d, dv, F, V = sz["width"], sz["heads"], sz["kv_heads"], sz["dim"], sz["vdim"], sz["ff"], sz["vocab"]
        toks = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(7)).tolist()
        cap = max(T, 8 * (ctx + 32 * (K + 2))) + 64
        res = {"config": sz}
        # -- the whole models: Kupelix, then Pubopel of the same width, heads and vocabulary
        cfg = SY.kupelix_config(**sz)
        model = CausalLM(KupelixConfig.model_validate(cfg), SY.kupelix_weights(cfg, WEIGHT_SEED, dev), dtype="bfloat16", device=dev,
                         max_tokens=cap, max_sequences=8, page_size=64, max_rows=R)
        res["kupelix"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        n_att = sz["kinds"].count("attention")
        L = len(sz["kinds"])
        per_layer = {"attention": H * d + G * d + G * dv + H, "hgrn2": 2 * H * d + H * dv,
                     "channel_delta": 2 * H * d + H * dv + H + 128}
        w_bytes = 2.0 * (sum(D * (per_layer[k] + F) + D * (H * dv + F) for k in sz["kinds"]) + D * V)
        state_bytes = 8.0 * H * d * dv * (L - n_att) + 4.0 * ctx * G * (d + dv) * n_att    # states read + written, keys + values read
        flops = sum(2.0 * T * D * (per_layer[k] + F) + 2.0 * T * D * (H * dv + F) for k in sz["kinds"]) + \
            n_att * 2.0 * H * (d + dv) * T * (T + 1) / 2 + (L - n_att) * 6.0 * T * H * d * dv + 2.0 * D * V
        res["kupelix"]["prefill"].update(model_tflops=flops / res["kupelix"]["prefill"]["ms"] / 1e9,
                                         frac_of_bf16_peak=flops / res["kupelix"]["prefill"]["ms"] / 1e9 / tf)
        b1 = res["kupelix"]["decode_b1"]
        b1.update(algorithmic_bytes=w_bytes + state_bytes, gb_per_s=(w_bytes + state_bytes) / b1["ms_per_step"] / 1e6,
                  frac_of_hbm_peak=(w_bytes + state_bytes) / b1["ms_per_step"] / 1e6 / hbm)
        model.engine.close()
        del model
        torch.cuda.empty_cache()
        pcfg = SY.pubopel_config(**psz)
        model = CausalLM(PubopelConfig.model_validate(pcfg), SY.pubopel_weights(pcfg, WEIGHT_SEED, dev), dtype="bfloat16", device=dev,
                         max_tokens=cap, max_sequences=8, page_size=64, max_rows=R)
        res["pubopel"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        model.engine.close()
        del model
        torch.cuda.empty_cache()

        # -- kernels alone: one-layer models, the mixer kernels on given projections (no products around them)
        kern = {}

        def one_layer(kind):
            c1 = SY.kupelix_config(**{**sz, "kinds": [kind], "vocab": 256, "ff": 8})
            return CausalLM(KupelixConfig.model_validate(c1), SY.kupelix_weights(c1, 3, dev), dtype="float32", device=dev,
                            max_tokens=8 * T + 64, max_sequences=8, page_size=64, max_rows=R)

        def timed_mixer(m1, n_seq, rows_each, start):
            """rows_each new rows for each of n_seq sequences that already hold `start` tokens (state appended each call)."""
            n_in = m1.layers[0].layer.n_in
            proj = torch.randn(n_seq * min(rows_each, R), n_in, device=dev) * 0.5
            seqs = [m1.state.open(f"s{i}") for i in range(n_seq)]
            for sq in seqs:
                m1.state.reserve(sq, start + rows_each)
            def run():
                for r0 in range(0, rows_each, R):
                    n = min(R, rows_each - r0)
                    m1.engine.op_mixer_kernels(0, proj[:n_seq * n], [(sq, n, start + r0) for sq in seqs])
            ms = _event_ms(run, 2, K, flush)
            for i in range(n_seq):
                m1.state.close(f"s{i}")
            return ms

        m1 = one_layer("attention")
        a_flops = 2.0 * H * (d + dv) * T * (T + 1) / 2
        ms_k = timed_mixer(m1, 1, T, 0)
        kern["attention_causal"] = {"T": T, "heads": H, "kv_heads": G, "dim": d, "vdim": dv, "kupelix_ms": ms_k,
                                    "kupelix_tflops_fp32": a_flops / ms_k / 1e9}
        ms_k = timed_mixer(m1, 8, 1, ctx)                        # eight decoding rows, each over ctx keys (written by the call before)
        kv_bytes = 8.0 * ctx * G * (d + dv) * 4
        kern["attention_decode_b8"] = {"context": ctx, "kupelix_ms": ms_k, "kupelix_gb_per_s": kv_bytes / ms_k / 1e6,
                                       "kupelix_frac_of_hbm_peak": kv_bytes / ms_k / 1e6 / hbm}
        m1.engine.close()
        full_cfg = SY.pubopel_config(**{**psz, "layers": 1, "window": None, "vocab": 256, "experts": 1, "top": 1, "expert_ff": 8,
                                        "shared_ff": None})
        full = CausalLM(PubopelConfig.model_validate(full_cfg), SY.pubopel_weights(full_cfg, 3, dev), dtype="float32", device=dev,
                        max_tokens=8 * T + 64, max_sequences=8, page_size=64, max_rows=R)
        qk = torch.randn(T, (H + G) * d, device=dev)

        def pub_attn(n_seq, rows_each, start):
            seqs = [full.state.open(f"s{i}") for i in range(n_seq)]
            for sq in seqs:
                full.state.reserve(sq, start + rows_each)
            def run():
                for r0 in range(0, rows_each, R):
                    n = min(R, rows_each - r0)
                    full.engine.op_attention(0, qk[:n_seq * n], [(sq, n, start + r0) for sq in seqs])
            ms = _event_ms(run, 2, K, flush)
            for i in range(n_seq):
                full.state.close(f"s{i}")
            return ms
        ms_p = pub_attn(1, T, 0)
        kern["attention_causal"].update(pubopel_ms=ms_p, pubopel_tflops_fp32=4.0 * d * H * T * (T + 1) / 2 / ms_p / 1e9)
        ms_p = pub_attn(8, 1, ctx)
        pk_bytes = 8.0 * ctx * G * 2 * d * 4
        kern["attention_decode_b8"].update(pubopel_ms=ms_p, pubopel_gb_per_s=pk_bytes / ms_p / 1e6,
                                           pubopel_frac_of_hbm_peak=pk_bytes / ms_p / 1e6 / hbm)
        full.engine.close()
        del full, m1
        torch.cuda.empty_cache()
        for kind in ("hgrn2", "channel_delta"):
            m1 = one_layer(kind)
            n_in = m1.layers[0].layer.n_in
            ent = {}
            for label, (n_seq, rows_each, start) in {"prefill_1x%d" % T: (1, T, 0), "prefill_8x512": (8, 512, 0),
                                                     "decode_b8": (8, 1, 64)}.items():
                ms_k = timed_mixer(m1, n_seq, rows_each, start)
                rows = n_seq * rows_each
                byt = rows * 4.0 * (n_in + H * dv) + n_seq * 8.0 * H * d * dv          # projections in, read-out, states in and out
                ent[label] = {"ms": ms_k, "rows_per_s": rows / ms_k * 1e3, "gb_per_s": byt / ms_k / 1e6,
                              "frac_of_hbm_peak": byt / ms_k / 1e6 / hbm,
                              "state_tflops_fp32": (6.0 if kind == "hgrn2" else 10.0) * rows * H * d * dv / ms_k / 1e9}
            kern[kind + "_recurrence"] = ent
            m1.engine.close()
            del m1
            torch.cuda.empty_cache()
        res["kernels"] = kern
        out[name] = res
    clocks = sampler.stop()
    print(json.dumps({"metric": "lm_layer_throughput", "design": "kupelix", "impl": "ours", "n_gpus": 1, "steps": K, "warmup": W,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
                      "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
                      "timing": "CUDA events, median; a 160 MB buffer is rewritten between timed iterations (L2 flush)",
                      "gpu_launches": launch_count() - launches0, "clocks": clocks, "lm": out}))


# ---- --lm --lm-design luketar: the Luketar design beside Kupelix and Pubopel at equal width, its mixers beside Kupelix's -----
LUKETAR_SIZES = {
    # the widths, head counts and vocabularies of LM_SIZES / KUPELIX_SIZES; a dense gated unit in the first layer and
    # Pubopel's expert sizes in the others; the cached latent is as wide as two of Kupelix's four key heads
    "w2048": dict(width=2048, kinds=["latent_attention", "mlstm", "latent_attention", "latent_attention"], heads=16, dim=128, vdim=128,
                  q_rank=768, kv_rank=256, ff=4096, experts=8, top=2, expert_ff=2048, shared_ff=4096, vocab=32768, streams=4),
    "w1024": dict(width=1024, kinds=["latent_attention", "mlstm", "latent_attention", "latent_attention"], heads=8, dim=128, vdim=128,
                  q_rank=384, kv_rank=128, ff=1024, experts=16, top=2, expert_ff=512, shared_ff=1024, vocab=16384, streams=4),
}


def run_lm_luketar(args) -> None:
    import torch
    from dia_tts_prune_b200 import synthetic as SY
    from dia_tts_prune_b200.lm_config import KupelixConfig, LuketarConfig, PubopelConfig
    from dia_tts_prune_b200.lm_engine import launch_count
    from dia_tts_prune_b200.lm_model import CausalLM

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        hbm, tf, src = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), "measured"
    except Exception:
        hbm, tf, src = 6650.0, 1590.0, "fallback"
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)             # > the 126 MB L2
    W, K = max(args.warmup, 3), max(args.steps, 3)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = launch_count()
    out = {}
    T, ctx, R = args.lm_prompt, args.lm_context, args.lm_rows
    for name in (args.lm_sizes.split(",") if args.lm_sizes else LUKETAR_SIZES):
        sz, ksz, psz = LUKETAR_SIZES[name], KUPELIX_SIZES[name], LM_SIZES[name]
        D, H, d, dv, V = sz["width"], sz["heads"], sz["dim"], sz["vdim"], sz["vocab"]
        rq, rk, s = sz["q_rank"], sz["kv_rank"], sz["streams"]
        toks = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(7)).tolist()
        cap = max(T, 8 * (ctx + 32 * (K + 2))) + 64
        res = {"config": sz}
        kw = dict(dtype="bfloat16", device=dev, max_tokens=cap, max_sequences=8, page_size=64, max_rows=R)
        cfg = SY.luketar_config(**sz)
        model = CausalLM(LuketarConfig.model_validate(cfg), SY.luketar_weights(cfg, WEIGHT_SEED, dev), **kw)
        res["luketar"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        kinds = sz["kinds"]
        n_att, L = kinds.count("latent_attention"), len(kinds)
        # products per token: stacked input projections, latent up-projections (the key / value ones per head in the latent
        # space), output projection, active feed-forward units
        att_cols = D * (rq + rk + H * dv) + rq * H * d + H * d * rk + H * rk * dv + H * dv * D
        mem_cols = D * (2 * H * d + 2 * H * dv + 2 * H) + H * dv * D
        ff_cols = [3 * D * sz["ff"]] + [3 * D * (sz["top"] * sz["expert_ff"] + sz["shared_ff"]) + D * sz["experts"]] * (L - 1)
        mix_cols = [att_cols if k == "latent_attention" else mem_cols for k in kinds]
        flops = 2.0 * T * (sum(mix_cols) + sum(ff_cols)) + n_att * 4.0 * H * rk * T * (T + 1) / 2 + \
            (L - n_att) * 4.0 * T * H * d * (dv + 1) + 2.0 * D * V
        w_bytes = 2.0 * (sum(mix_cols) + sum(ff_cols) + D * V)
        state_bytes = 4.0 * ctx * rk * n_att + 8.0 * H * d * (dv + 1) * (L - n_att) + 8.0 * 2 * L * s * D
        res["luketar"]["prefill"].update(model_tflops=flops / res["luketar"]["prefill"]["ms"] / 1e9,
                                         frac_of_bf16_peak=flops / res["luketar"]["prefill"]["ms"] / 1e9 / tf)
        b1 = res["luketar"]["decode_b1"]
        b1.update(algorithmic_bytes=w_bytes + state_bytes, gb_per_s=(w_bytes + state_bytes) / b1["ms_per_step"] / 1e6,
                  frac_of_hbm_peak=(w_bytes + state_bytes) / b1["ms_per_step"] / 1e6 / hbm)
        model.engine.close()
        del model
        torch.cuda.empty_cache()
        kcfg = SY.kupelix_config(**ksz)
        model = CausalLM(KupelixConfig.model_validate(kcfg), SY.kupelix_weights(kcfg, WEIGHT_SEED, dev), **kw)
        res["kupelix"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        model.engine.close()
        del model
        torch.cuda.empty_cache()
        pcfg = SY.pubopel_config(**psz)
        model = CausalLM(PubopelConfig.model_validate(pcfg), SY.pubopel_weights(pcfg, WEIGHT_SEED, dev), **kw)
        res["pubopel"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        model.engine.close()
        del model
        torch.cuda.empty_cache()

        # -- mixers alone (projections, kernels, output projection; no feed-forward): one-layer models of either design
        def timed(m1, n_seq, rows_each, start):
            h = torch.randn(n_seq * min(rows_each, R), D, device=dev)
            seqs = [m1.state.open(f"s{i}") for i in range(n_seq)]
            for sq in seqs:
                m1.state.reserve(sq, start + rows_each)
            def run():
                for r0 in range(0, rows_each, R):
                    n = min(R, rows_each - r0)
                    m1.engine.op_mixer(0, h[:n_seq * n], [(sq, n, start + r0) for sq in seqs])
            ms = _event_ms(run, 2, K, flush)
            for i in range(n_seq):
                m1.state.close(f"s{i}")
            return ms

        kw1 = dict(dtype="bfloat16", device=dev, max_tokens=8 * T + 64, max_sequences=8, page_size=64, max_rows=R)
        mixers = {}
        for kind, twin in (("latent_attention", "attention"), ("mlstm", "hgrn2")):
            c1 = SY.luketar_config(**{**sz, "kinds": [kind], "vocab": 256, "ff": 0, "experts": 0})
            m1 = CausalLM(LuketarConfig.model_validate(c1), SY.luketar_weights(c1, 3, dev), **kw1)
            k1 = SY.kupelix_config(**{**ksz, "kinds": [twin], "vocab": 256, "ff": 8})
            m2 = CausalLM(KupelixConfig.model_validate(k1), SY.kupelix_weights(k1, 3, dev), **kw1)
            ent = {}
            for label, (n_seq, rows_each, start) in {"prefill_1x%d" % T: (1, T, 0), "decode_b8": (8, 1, ctx)}.items():
                ent[label] = {"luketar_ms": timed(m1, n_seq, rows_each, start), "kupelix_" + twin + "_ms": timed(m2, n_seq, rows_each, start)}
            if kind == "latent_attention":
                ent["prefill_1x%d" % T].update(luketar_attention_flops=4.0 * H * rk * T * (T + 1) / 2,
                                               kupelix_attention_flops=2.0 * H * (d + dv) * T * (T + 1) / 2)
                ent["decode_b8"].update(luketar_cache_bytes=8.0 * ctx * rk * 4, kupelix_cache_bytes=8.0 * ctx * ksz["kv_heads"] * (d + dv) * 4)
            mixers[kind] = ent
            m1.engine.close()
            m2.engine.close()
            del m1, m2
            torch.cuda.empty_cache()
        res["mixers"] = mixers
        out[name] = res
    clocks = sampler.stop()
    print(json.dumps({"metric": "lm_layer_throughput", "design": "luketar", "impl": "ours", "n_gpus": 1, "steps": K, "warmup": W,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
                      "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
                      "timing": "CUDA events, median; a 160 MB buffer is rewritten between timed iterations (L2 flush)",
                      "gpu_launches": launch_count() - launches0, "clocks": clocks, "lm": out}))


# ---- --lm --lm-design fipadra: the Fipadra design beside Luketar at equal width, its mixers beside their likes -----------------
FIPADRA_SIZES = {
    # the widths, head counts, latent sizes, expert sizes and vocabularies of LUKETAR_SIZES; a query / key head of 96 plain + 32
    # turned channels (128 as there), a window as long as the decode context, a squared-relu unit with the parameter count of
    # Luketar's gated one, two identity experts beside the eight / sixteen routed ones, two groups of which one is kept
    "w2048": dict(width=2048, kinds=["delta", "latent_attention", "retention", "latent_attention"], heads=16, kv_heads=4, dim=128,
                  vdim=128, q_rank=768, kv_rank=256, rot_dim=32, window=1024, taps=4, ff=6144, experts=8, top=2, identity=2,
                  groups=(2, 1), expert_ff=2048, shared_ff=4096, vocab=32768),
    "w1024": dict(width=1024, kinds=["delta", "latent_attention", "retention", "latent_attention"], heads=8, kv_heads=2, dim=128,
                  vdim=128, q_rank=384, kv_rank=128, rot_dim=32, window=1024, taps=4, ff=1536, experts=16, top=2, identity=2,
                  groups=(2, 1), expert_ff=512, shared_ff=1024, vocab=16384),
}


def _fipadra_config(sz: dict) -> dict:
    """The model of a size entry: attention heads are [dim - rot_dim plain | rot_dim turned], the other mixers use `dim`."""
    from dia_tts_prune_b200 import synthetic as SY
    cfg = SY.fipadra_config(**sz)
    for lc in cfg["layers"]:
        if lc["type"] == "latent_attention":
            lc["mixer"]["dim"] = sz["dim"] - sz["rot_dim"]
    return cfg


def run_lm_fipadra(args) -> None:
    import torch
    from dia_tts_prune_b200 import synthetic as SY
    from dia_tts_prune_b200.lm_config import FipadraConfig, KupelixConfig, LuketarConfig
    from dia_tts_prune_b200.lm_engine import launch_count
    from dia_tts_prune_b200.lm_model import CausalLM

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        hbm, tf, src = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), "measured"
    except Exception:
        hbm, tf, src = 6650.0, 1590.0, "fallback"
    flush = torch.zeros(160 << 20, dtype=torch.uint8, device=dev)             # > the 126 MB L2
    W, K = max(args.warmup, 3), max(args.steps, 3)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = launch_count()
    out = {}
    T, ctx, R = args.lm_prompt, args.lm_context, args.lm_rows
    for name in (args.lm_sizes.split(",") if args.lm_sizes else FIPADRA_SIZES):
        sz, lsz, ksz = FIPADRA_SIZES[name], LUKETAR_SIZES[name], KUPELIX_SIZES[name]
        D, H, G, d, dv, V = sz["width"], sz["heads"], sz["kv_heads"], sz["dim"], sz["vdim"], sz["vocab"]
        rq, rk, dr, win = sz["q_rank"], sz["kv_rank"], sz["rot_dim"], sz["window"]
        toks = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(7)).tolist()
        cap = max(T, 8 * (ctx + 32 * (K + 2))) + 64
        res = {"config": {k: (list(v) if isinstance(v, tuple) else v) for k, v in sz.items()}}
        kw = dict(dtype="bfloat16", device=dev, max_tokens=cap, max_sequences=8, page_size=64, max_rows=R)
        cfg = _fipadra_config(sz)
        model = CausalLM(FipadraConfig.model_validate(cfg), SY.fipadra_weights(cfg, WEIGHT_SEED, dev), **kw)
        res["fipadra"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        kinds = sz["kinds"]
        # products per token and mixer: stacked input projections, (latent up-projections,) output projection
        cols = {"delta": D * (2 * G * d + 2 * H * dv + 2 * H) + H * dv * D,
                "retention": D * (2 * H * d + 2 * H * dv) + H * dv * D,
                "latent_attention": D * (rq + rk + dr) + rq * H * d + H * (d - dr) * rk + H * rk * dv + H * dv * D}
        moe_cols = 3 * D * (sz["top"] * sz["expert_ff"] + sz["shared_ff"]) + D * (sz["experts"] + sz["identity"] + 1)
        ff_cols = [moe_cols if n % 2 else 2 * D * sz["ff"] for n in range(len(kinds))]
        keys = sum(min(t + 1, win) for t in range(T))             # (query, key) pairs of a windowed prompt
        mixer_flops = {"delta": 6.0 * T * H * d * dv, "retention": 4.0 * T * H * d * dv,
                       "latent_attention": 2.0 * H * (2 * rk + dr) * keys}
        flops = 2.0 * T * (sum(cols[k] for k in kinds) + sum(ff_cols)) + sum(mixer_flops[k] for k in kinds) + 2.0 * D * V
        w_bytes = 2.0 * (sum(cols[k] for k in kinds) + sum(ff_cols) + D * V)
        state = {"delta": 8.0 * H * d * dv, "retention": 8.0 * H * d * dv, "latent_attention": 4.0 * min(ctx, win) * (rk + dr)}
        state_bytes = sum(state[k] for k in kinds) + 8.0 * len(kinds) * D
        pf, b1 = res["fipadra"]["prefill"], res["fipadra"]["decode_b1"]
        pf.update(model_tflops=flops / pf["ms"] / 1e9, frac_of_bf16_peak=flops / pf["ms"] / 1e9 / tf)
        b1.update(algorithmic_bytes=w_bytes + state_bytes, gb_per_s=(w_bytes + state_bytes) / b1["ms_per_step"] / 1e6,
                  frac_of_hbm_peak=(w_bytes + state_bytes) / b1["ms_per_step"] / 1e6 / hbm)
        model.engine.close()
        del model
        torch.cuda.empty_cache()
        lcfg = SY.luketar_config(**lsz)
        model = CausalLM(LuketarConfig.model_validate(lcfg), SY.luketar_weights(lcfg, WEIGHT_SEED, dev), **kw)
        res["luketar"] = _lm_prefill_decode(model, toks, T, ctx, W, K, flush)
        model.engine.close()
        del model
        torch.cuda.empty_cache()

        # -- mixers alone (projections, kernels, output projection; no feed-forward): one-layer models of either design
        def timed(m1, n_seq, rows_each, start):
            h = torch.randn(n_seq * min(rows_each, R), D, device=dev)
            seqs = [m1.state.open(f"s{i}") for i in range(n_seq)]
            for sq in seqs:
                m1.state.reserve(sq, start + rows_each)
            def run():
                for r0 in range(0, rows_each, R):
                    n = min(R, rows_each - r0)
                    m1.engine.op_mixer(0, h[:n_seq * n], [(sq, n, start + r0) for sq in seqs])
            ms = _event_ms(run, 2, K, flush)
            for i in range(n_seq):
                m1.state.close(f"s{i}")
            return ms

        kw1 = dict(dtype="bfloat16", device=dev, max_tokens=8 * T + 64, max_sequences=8, page_size=64, max_rows=R)
        mixers = {}
        for kind, (twin_design, twin) in (("latent_attention", ("luketar", "latent_attention")), ("retention", ("luketar", "mlstm")),
                                          ("delta", ("kupelix", "channel_delta"))):
            c1 = _fipadra_config({**sz, "kinds": [kind], "vocab": 256, "ff": 0, "experts": 0})
            m1 = CausalLM(FipadraConfig.model_validate(c1), SY.fipadra_weights(c1, 3, dev), **kw1)
            if twin_design == "luketar":
                c2 = SY.luketar_config(**{**lsz, "kinds": [twin], "vocab": 256, "ff": 0, "experts": 0, "streams": None})
                m2 = CausalLM(LuketarConfig.model_validate(c2), SY.luketar_weights(c2, 3, dev), **kw1)
            else:
                c2 = SY.kupelix_config(**{**ksz, "kinds": [twin], "vocab": 256, "ff": 8})
                m2 = CausalLM(KupelixConfig.model_validate(c2), SY.kupelix_weights(c2, 3, dev), **kw1)
            ent = {}
            for label, (n_seq, rows_each, start) in {"prefill_1x%d" % T: (1, T, 0), "prefill_8x%d" % (T // 8): (8, T // 8, 0),
                                                     "decode_b8": (8, 1, ctx)}.items():
                ent[label] = {"fipadra_ms": timed(m1, n_seq, rows_each, start),
                              f"{twin_design}_{twin}_ms": timed(m2, n_seq, rows_each, start)}
            if kind == "latent_attention":
                ent["prefill_1x%d" % T].update(fipadra_attention_flops=2.0 * H * (2 * rk + dr) * keys,
                                               luketar_attention_flops=4.0 * H * lsz["kv_rank"] * T * (T + 1) / 2)
            mixers[kind] = ent
            m1.engine.close()
            m2.engine.close()
            del m1, m2
            torch.cuda.empty_cache()
        res["mixers"] = mixers
        out[name] = res
    clocks = sampler.stop()
    print(json.dumps({"metric": "lm_layer_throughput", "design": "fipadra", "impl": "ours", "n_gpus": 1, "steps": K, "warmup": W,
                      "dtype": "bf16", "data": "synthetic (random weights, random token ids)",
                      "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src},
                      "timing": "CUDA events, median; a 160 MB buffer is rewritten between timed iterations (L2 flush)",
                      "gpu_launches": launch_count() - launches0, "clocks": clocks, "lm": out}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-decode-steps", type=int, default=12, help="decode steps of the cpu_baseline sample")
    ap.add_argument("--ref-decode-steps", type=int, default=4, help="decode steps per reference-arm bench step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--variant", default="dense", choices=sorted(VARIANTS),
                    help="dense = BASELINE.json configs[1] (the headline); the others are configs[3]")
    ap.add_argument("--prune-amount", type=float, default=0.5, help="mlp-pruned: fraction of hidden neurons removed")
    ap.add_argument("--utterances", type=int, default=0,
                    help="BASELINE.json configs[4]: run this many synthetic transcripts sharded over the GPUs instead of "
                         "the headline single-transcript workload")
    ap.add_argument("--max-tokens", type=int, default=MAX_TOKENS, help="--utterances mode: frames per utterance")
    ap.add_argument("--per-launch", type=int, default=8, help="utterances decoded together in one kernel launch (1..8)")
    ap.add_argument("--batch-utterances", type=int, default=64,
                    help="headline mode: also run configs[4] with this many transcripts (0 = skip) and print it as `batch`")
    ap.add_argument("--lm", action="store_true",
                    help="instead of the headline workload: prefill / decode throughput of the decoder-only language-model path "
                         "(Pubopel, random weights) at layer sizes of a real model, beside Dia's kernels at equal size")
    ap.add_argument("--lm-design", default="pubopel", choices=["pubopel", "kupelix", "luketar", "fipadra"],
                    help="--lm: the design that is measured (kupelix: beside Pubopel at equal width, and its kernels beside Pubopel's; "
                         "luketar: beside Kupelix and Pubopel at equal width, and its mixers beside Kupelix's; fipadra: beside Luketar at equal "
                         "width, and its mixers beside their likes in Luketar and Kupelix)")
    ap.add_argument("--lm-sizes", default="", help="--lm: comma-separated subset of " + ",".join(LM_SIZES))
    ap.add_argument("--lm-prompt", type=int, default=4096, help="--lm: prompt tokens of the prefill measurement")
    ap.add_argument("--lm-rows", type=int, default=4096, help="--lm: most rows of one engine step (longer prompts run in portions)")
    ap.add_argument("--lm-context", type=int, default=1024, help="--lm: tokens each sequence holds before the decode measurement")
    args = ap.parse_args()
    if args.lm:
        {"kupelix": run_lm_kupelix, "luketar": run_lm_luketar, "fipadra": run_lm_fipadra}.get(args.lm_design, run_lm)(args)
        return
    if args.impl == "reference":
        run_reference(args)
        return
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        import socket
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
        raise SystemExit(subprocess.call(cmd))
    if args.utterances > 0:
        run_batch(args)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
