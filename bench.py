#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s) of Mistral-7B-architecture NF4 QLoRA.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N ...            # the unmodified reference (if installable)

Model and data follow the benchmark definition: 32 layers, hidden 4096, 32 heads / 8 KV heads, SwiGLU 14336,
vocab 32000, RoPE theta 1e6; base weights random normal(0, 0.02) quantised to NF4 (block 64, double-quantised
scales); LoRA r=16, alpha=16 on q/k/v/o in bf16; per-device batch 4 x 4096 uniform-random tokens packed
padding-free from documents of length uniform[128, 4096]; fused CE / RMSNorm / RoPE kernels on.  Every step is
forward + backward + AdamW step.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

BASELINE_TOK_S = 4128.0  # Mistral-7B NF4 QLoRA + fused ops, 1 x A100-80GB, bs4 (reference CSV a100_80gb.csv:82)


def reference_arm(args) -> int:
    """Run the unmodified reference from baseline/_ref through its own public API; print why when that is impossible.

    The attempt is real: a child process with baseline/_ref first on its path imports the reference's framework
    package and its benchmark's trainer entry point, exactly what ``scripts/benchmarks/benchmark.py`` of the reference
    would launch.  On this image the import stops at the first missing dependency (peft / accelerate / trl /
    bitsandbytes are not installed and cannot be: no network, not in the wheelhouse); that error is reported."""
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "fms_acceleration")):
        reason = ("baseline/_ref holds no copy of the reference (python -m fms_acceleration_b200.baseline."
                  "install_reference <checkout> was not run on this checkout)")
    else:
        probe = ("import sys; sys.path.insert(0, sys.argv[1]); "
                 "import fms_acceleration; from fms_acceleration import AccelerationFramework; "
                 "import fms_acceleration_peft, fms_acceleration_foak; import tuning.sft_trainer")
        res = subprocess.run([sys.executable, "-c", probe, ref_dir], capture_output=True, text=True, cwd=ref_dir,
                             env={k: v for k, v in os.environ.items() if k != "PYTHONPATH"})
        if res.returncode == 0:
            reason = ("the reference imports, but its benchmark downloads the model and the dataset from the network, "
                      "which this machine does not have")
        else:
            last = [ln for ln in res.stderr.strip().splitlines() if ln.strip()]
            reason = ("the reference's public API does not import on this image: "
                      + (last[-1] if last else f"exit code {res.returncode}"))[:300]
    if int(os.environ.get("RANK", "0")) == 0:  # one line per job, also when launched with one process per GPU
        print(json.dumps({"impl": "reference", "unavailable": reason.replace("\n", " ")}), flush=True)
    return 0


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(gpu_index)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.tmp.read().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.tmp.name)
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


# ------------------------------------------------------------------------------------------- benchmark configs
# name -> (metric label, model preset, per-device batch, sequence length, published A100 number or None)
CONFIGS = {
    "mistral-qlora": ("train tokens/sec, Mistral-7B NF4 QLoRA", "mistral-7b", 4, 4096, 4128.0),
    "granite-moe": ("train tokens/sec, Granite-3B-A800M ScatterMoE full fine-tune", "granite-3b-a800m", 8, 2048, 6216.0),
    "llama70b-gptq": ("train tokens/sec, Llama-2-70B GPTQ-LoRA", "llama2-70b", 1, 4096, 496.0),
    "mamba-cp": ("train tokens/sec, Mamba2-2.7B context parallel", "mamba2-2.7b", 1, 65536, None),
}
FOAK = {"fused_lora": True, "fast_loss": "fused_ce_liger", "fast_rms_layernorm": True, "fast_rope_embeddings": True}


def framework_config(name: str, world: int, impl: str = "b200") -> dict:
    cfg = _framework_config(name, world)
    if impl == "baseline":
        # the comparison arm runs the library kernels: the fused-ops plugin stays out
        def strip(d):
            return {k: strip(v) for k, v in d.items() if k != "fused_ops_and_kernels"} if isinstance(d, dict) else d

        cfg = strip(cfg)
    return cfg


def _framework_config(name: str, world: int) -> dict:
    if name == "mistral-qlora":
        return {"peft": {"quantization": {"bitsandbytes": {"quant_type": "nf4", "no_peft_model": False},
                                          "fused_ops_and_kernels": dict(FOAK, base_layer="bitsandbytes")}},
                "training": {"attention": {"padding_free": {"method": "huggingface"}}}}
    if name == "llama70b-gptq":
        return {"peft": {"quantization": {"auto_gptq": {"kernel": "triton_v2", "from_quantized": True},
                                          "fused_ops_and_kernels": dict(FOAK, base_layer="auto_gptq")}},
                "training": {"attention": {"padding_free": {"method": "huggingface"}}}}
    if name == "granite-moe":
        ep = max(d for d in (1, 2, 4, 8) if world % d == 0 and d <= world)
        foak = {k: v for k, v in FOAK.items() if k != "fused_lora"}
        return {"training": {"moe": {"scattermoe": {"ep_degree": ep}},
                             "attention": {"padding_free": {"method": "huggingface"}},
                             "fused_ops_and_kernels": foak}}
    if name == "mamba-cp":
        cfg = {"training": {"fused_ops_and_kernels": {k: v for k, v in FOAK.items() if k != "fused_lora"}}}
        if world > 1:
            cfg["training"]["mamba"] = {"cp": {"degree": world, "mamba_impl": "allgather", "mamba_recompute": False}}
        return cfg
    raise KeyError(name)


def make_batches(name, cfg, batch, seq, rank, world, n_batches):
    import torch

    from fms_acceleration_b200.trainer import synthetic_packed_batch

    if name != "mamba-cp":
        lo = min(128, seq)
        return [synthetic_packed_batch(cfg.vocab_size, batch, seq, (lo, seq), seed=1000 * rank + i)
                for i in range(n_batches)], batch * seq * world
    # one sequence of `seq` tokens split evenly over the context-parallel ranks (same tokens on every rank's view)
    out = []
    per = seq // world
    for i in range(n_batches):
        g = torch.Generator().manual_seed(77 + i)
        ids = torch.randint(0, cfg.vocab_size, (1, seq), generator=g, dtype=torch.int64)
        sl = ids[:, rank * per:(rank + 1) * per].contiguous()
        b = {"input_ids": sl, "labels": sl.clone()}
        if torch.cuda.is_available():
            b = {k: v.pin_memory() for k, v in b.items()}
        out.append(b)
    return out, seq


def run_config(name: str, args, ctx, impl: str = "b200") -> dict:
    """Build the model through the framework's public lifecycle and time `args.steps` optimizer steps.

    ``impl="baseline"``: the same model, data, optimizer and trainer, executed through library kernels (cuBLAS,
    flash-attn, NCCL) and the reference's Triton kernels loaded by file path (fms_acceleration_b200/baseline)."""
    import torch
    import torch.distributed as dist
    import yaml

    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.compat import Accelerator
    from fms_acceleration_b200.framework import AccelerationFramework
    from fms_acceleration_b200.models.builder import build_model, resolve_config
    from fms_acceleration_b200.nn import LoraConfig
    from fms_acceleration_b200.trainer import TrainArgs, Trainer, to_device

    rank, local_rank, world, dev = ctx["rank"], ctx["local_rank"], ctx["world"], ctx["dev"]
    metric, preset, batch, seq, published = CONFIGS[name]
    batch = args.batch or batch
    seq = args.seq or seq
    cfg = resolve_config(args.model or preset)
    if args.layers:
        cfg.num_hidden_layers = args.layers
    dtype = torch.float16 if name == "llama70b-gptq" and args.fp16 else torch.bfloat16
    with tempfile.TemporaryDirectory() as td:
        cfg_path = os.path.join(td, "accel.yaml")
        with open(cfg_path, "w", encoding="utf-8") as fh:
            yaml.safe_dump({"plugins": framework_config(name, world, impl)}, fh)
        AccelerationFramework.reset()
        framework = AccelerationFramework(cfg_path)
    train_args = TrainArgs(per_device_train_batch_size=batch, learning_rate=1e-4 if "lora" in metric.lower() else 2e-5,
                           bf16=dtype == torch.bfloat16, fp16=dtype == torch.float16, max_seq_length=seq,
                           padding_free=name != "mamba-cp", world_size=world,
                           parallel_mode="DISTRIBUTED" if world > 1 else "NOT_DISTRIBUTED")
    if impl == "baseline":
        os.environ["FMSB_ENGINE_BACKEND"] = "library"
        os.environ["FMSB_MOE_BACKEND"] = "library"
    else:
        os.environ.pop("FMSB_ENGINE_BACKEND", None)
        os.environ.pop("FMSB_MOE_BACKEND", None)
    torch.manual_seed(1234)
    if framework.requires_custom_loading:
        model = framework.model_loader(cfg, torch_dtype=dtype, device=dev)
    else:
        model = build_model(cfg, device=dev, dtype=dtype, seed=1234)
    peft_config = None
    if name in ("mistral-qlora", "llama70b-gptq"):
        peft_config = LoraConfig(r=16, lora_alpha=16, lora_dropout=0.0,
                                 target_modules=["q_proj", "k_proj", "v_proj", "o_proj"])
    model, _ = framework.augmentation(model, train_args, modifiable_args=(peft_config,))
    accelerator = Accelerator(device=dev)
    callbacks = framework.get_callbacks_and_ready_for_train(model, accelerator)
    engine = getattr(accelerator, "engine", None)
    if engine is None and world > 1:
        from fms_acceleration_b200.parallel.engine import install_engine

        engine = install_engine(model, accelerator, shard_frozen=False)
    runner = model
    if impl == "baseline":
        from fms_acceleration_b200.baseline import BaselineRunner

        runner = BaselineRunner(model, gradient_checkpointing=args.baseline_checkpointing)
    elif args.gradient_checkpointing or (name == "mamba-cp" and seq // world > 8192):
        # a 65536-token sequence on 2 or 4 ranks does not fit with every layer's activations resident
        train_args.gradient_checkpointing = True
    trainer = Trainer(runner, train_args, engine=engine, callbacks=callbacks)

    n_batches = 4
    host_batches, tokens_per_step = make_batches(name, cfg, batch, seq, rank, world, n_batches)
    dev_batches = [to_device(b, dev) for b in host_batches]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(args.warmup):
        trainer.train_step(dev_batches[i % n_batches])
    barrier()
    NV.check_status()

    # ---- device-timed region: inputs already on the device
    sampler = ClockSampler(local_rank) if rank == 0 else None
    calls0 = NV.launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        trainer.train_step(dev_batches[i % n_batches])
    end.record()
    barrier()
    ms = start.elapsed_time(end)
    launches = NV.launch_count() - calls0
    clocks = sampler.stop() if sampler else None
    NV.check_status()

    # ---- end-to-end region: pinned host batch -> device every step, loss read back every step
    h2d = sum(v.numel() * v.element_size() for v in host_batches[0].values())
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e_start.record()
    last = 0.0
    for i in range(args.steps):
        loss = trainer.train_step(host_batches[i % n_batches])
        last = float(loss.item())
    e_end.record()
    barrier()
    e2e_ms_local = e_start.elapsed_time(e_end)

    kernel_table = None
    if getattr(args, "kernel_table", False) and rank == 0 or (getattr(args, "kernel_table", False) and world > 1):
        # device time per kernel over two more steps (torch.profiler / CUPTI; not part of any timed region)
        from torch.profiler import ProfilerActivity, profile

        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for i in range(2):
                trainer.train_step(dev_batches[i % n_batches])
            torch.cuda.synchronize()
        evs = sorted((e for e in prof.key_averages() if e.device_time_total > 0), key=lambda e: -e.device_time_total)
        total = sum(e.device_time_total for e in evs)
        kernel_table = {"device_ms_per_step": total / 2e3,
                        "top": [{"kernel": e.key[:100], "ms_per_step": round(e.device_time_total / 2e3, 3),
                                 "launches_per_step": e.count // 2} for e in evs[:25]]}

    t = torch.tensor([ms, e2e_ms_local], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    par = {"mistral-qlora": f"fsdp{world}", "llama70b-gptq": f"fsdp{world}",
           "granite-moe": f"ep{_framework_config(name, world)['training']['moe']['scattermoe']['ep_degree']}"
                          f"xdp{world}" if name == "granite-moe" else "", "mamba-cp": f"cp{world}"}[name]
    line = {
        "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if name == "mamba-cp" else "weak",
        "vs_baseline": (value / world / published) if published else None,
        "dtype": "fp16" if dtype == torch.float16 else "bf16",
        "data": "synthetic uniform-random tokens, random-init weights of the named architecture",
        "config": {"model": (args.model or preset) + ("" if not args.layers else f" (INVALID: {args.layers} layers)"),
                   "global_batch": batch * world if name != "mamba-cp" else 1, "seq_len": seq,
                   "parallelism": par if world > 1 else "single",
                   "l2": "step working set (tens of GB) far exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": launches,
        "final_loss": last,
        "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30,
    }
    if kernel_table is not None:
        line["kernel_table"] = kernel_table
    if impl == "baseline":
        from fms_acceleration_b200.baseline import reference_kernels_status

        line["impl"] = "baseline"
        line["kernels"] = reference_kernels_status()
        line["config"]["gradient_checkpointing"] = bool(args.baseline_checkpointing)
    else:
        line["config"]["gradient_checkpointing"] = bool(train_args.gradient_checkpointing)
        line["config"]["optimizer_state"] = "sharded over the ranks (ZeRO-1)" if getattr(
            trainer.optimizer, "sharded_state_dict", None) else "replicated"
    if name == "granite-moe" and impl != "baseline":
        from fms_acceleration_b200.ops import moe as MOE

        chunks = max(1, len(MOE.MoEContext._shared) and next(iter(MOE.MoEContext._shared.values())).C or 1)
        need = MOE.MoEContext.max_rows_needed(dev) / float(-(-batch * seq // chunks) * cfg.num_experts_per_tok)
        line["config"]["moe_rows_needed_over_balanced"] = round(need, 3)
        line["config"]["moe_chunks"] = chunks
        line["config"]["moe_rows_dropped_events"] = MOE.overflow_count(dev, reset=True)
        MOE.MoEContext._shared.clear()
    if name == "mistral-qlora":
        line["config"].update({"lora": "r16 a16 qkvo", "packing": "padding-free docs U[128,4096]"})
        line["vs_baseline"] = value / world / published  # published number is per device
    # release everything before another configuration is built in the same process
    del trainer, model, runner, dev_batches, engine, accelerator, callbacks
    import gc

    gc.collect()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    return line


def baseline_summary(name: str, args, ctx) -> dict:
    """Time the library-kernel arm of one configuration in the same process and boil it down to a few fields."""
    try:
        full = run_config(name, args, ctx, impl="baseline")
        return {"what": "same model, data, optimizer and trainer through cuBLAS torch.matmul, the installed flash-attn, "
                        "NCCL and the reference's Triton kernels loaded by file path; NOT the reference's public API",
                "value": full["value"], "unit": full["unit"], "ms_per_step": full["ms_per_step"],
                "e2e_value": full["e2e"]["value"], "final_loss": full["final_loss"], "kernels": full.get("kernels"),
                "gradient_checkpointing": full["config"].get("gradient_checkpointing"),
                "peak_mem_gb": full["peak_mem_gb"], "clocks": full["clocks"]}
    except Exception as exc:  # the product number must survive a failure of the comparison arm
        import traceback

        tb = traceback.format_exc().strip().splitlines()
        return {"error": f"{type(exc).__name__}: {exc}"[:300], "where": tb[-3:] if len(tb) >= 3 else tb}


def selfcheck(ctx) -> dict:
    """A few seconds of multi-GPU correctness before anything is timed: this package's peer-memory kernels against the
    library collectives on the same data (all-reduce; one expert-parallel mixture-of-experts layer, forward and input
    gradient, against the all_to_all form)."""
    import torch
    import torch.distributed as dist

    from fms_acceleration_b200 import _native as NV
    from fms_acceleration_b200.ops import moe as MOE
    from fms_acceleration_b200.parallel.symm import Communicator, SymmBuffer
    from fms_acceleration_b200.plugins.moe.utils.scattermoe import ScatterMoE

    rank, world, dev = ctx["rank"], ctx["world"], ctx["dev"]
    out = {}
    comm = Communicator()
    n = world * 8 * 4096
    bucket = SymmBuffer(n * 2)
    torch.manual_seed(10 + rank)
    x = torch.randn(n, device=dev).bfloat16()
    bucket.view(0, n, torch.bfloat16).copy_(x)
    comm.barrier(0)
    comm.allreduce_(bucket, n, torch.bfloat16)
    ref = x.float()
    dist.all_reduce(ref)
    out["allreduce_max_abs_err"] = float((bucket.view(0, n, torch.bfloat16).float() - ref / world).abs().max())
    E = 8 if 8 % world == 0 else 2 * world
    H, I_, k, T = 512, 256, 2, 1024
    res = []
    for backend in ("fused", "library"):
        MOE.MoEContext._shared.clear()
        m = ScatterMoE(H, "silu", I_, E, top_k=k, dtype=torch.bfloat16, device=dev, ep_group=dist.group.WORLD,
                       token_budget=T)
        m.backend = backend
        with torch.no_grad():
            torch.manual_seed(5)
            m.router.weight.normal_(0, 0.05)
            torch.manual_seed(11 + rank)
            for w in (m.w1, m.w2, m.w3):
                w.weight.normal_(0, 0.05)
        torch.manual_seed(50 + rank)
        xi = (torch.randn(T, H, device=dev) * 0.5).bfloat16().requires_grad_()
        o, _ = m(xi)
        o.float().square().sum().backward()
        res.append((o.detach().float(), xi.grad.float()))
    MOE.MoEContext._shared.clear()
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp(min=1e-9))
    out["moe_ep_fwd_rel_err_vs_all_to_all"] = rel(res[0][0], res[1][0])
    out["moe_ep_dx_rel_err_vs_all_to_all"] = rel(res[0][1], res[1][1])
    NV.check_status()
    t = torch.tensor([out["allreduce_max_abs_err"], out["moe_ep_fwd_rel_err_vs_all_to_all"],
                      out["moe_ep_dx_rel_err_vs_all_to_all"]], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    out = {k_: float(v) for k_, v in zip(out, t.tolist())}
    out["ok"] = bool(out["allreduce_max_abs_err"] < 0.05 and out["moe_ep_fwd_rel_err_vs_all_to_all"] < 3e-2
                     and out["moe_ep_dx_rel_err_vs_all_to_all"] < 3e-2)
    out["ranks"] = world
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default="mistral-qlora", choices=sorted(CONFIGS))
    ap.add_argument("--also", nargs="*", default=None, choices=sorted(CONFIGS),
                    help="further configurations to time in the same run (reported under 'secondary'); default: "
                         "granite-moe next to the headline configuration")
    ap.add_argument("--model", default=None, help="override the model preset of the configuration")
    ap.add_argument("--batch", type=int, default=0, help="per-device batch (0: the configuration's)")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--fp16", action="store_true")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (result marked invalid)")
    ap.add_argument("--no-baseline", action="store_true", help="skip the library-kernel comparison arm")
    ap.add_argument("--baseline-checkpointing", action="store_true",
                    help="run the comparison arm with activation checkpointing (the reference's benchmark default)")
    ap.add_argument("--gradient-checkpointing", action="store_true", help="activation checkpointing in the product arm")
    ap.add_argument("--no-selfcheck", action="store_true")
    ap.add_argument("--kernel-table", action="store_true",
                    help="after the timed regions, profile two more steps and report device time per kernel")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    import fms_acceleration_b200.plugins  # registers the plugins  # noqa: F401

    ctx = {"rank": rank, "local_rank": local_rank, "world": world, "dev": dev}
    check = None
    if world > 1 and not args.no_selfcheck:
        try:
            check = selfcheck(ctx)
        except Exception as exc:
            check = {"ok": False, "error": f"{type(exc).__name__}: {exc}"[:300]}
    line = run_config(args.config, args, ctx)
    if check is not None:
        line["selfcheck"] = check
    with_baseline = {"mistral-qlora", "granite-moe"} if not args.no_baseline else set()
    if args.config in with_baseline:
        line["baseline_backend"] = baseline_summary(args.config, args, ctx)
    if args.also is not None:
        also = args.also
    elif args.config == "mistral-qlora" and not args.layers and not args.model:
        # the other benchmark configurations, so that one run records all of them (on one GPU the context-parallel
        # configuration is the same 65536-token sequence without a split: the strong-scaling reference)
        also = ["granite-moe", "llama70b-gptq", "mamba-cp"]
    else:
        also = []
    secondary = []
    for name in also:
        if name == args.config:
            continue
        sub = argparse.Namespace(**vars(args))
        sub.batch, sub.seq, sub.model = 0, 0, None
        try:
            sec = run_config(name, sub, ctx)
            if name in with_baseline:
                sec["baseline_backend"] = baseline_summary(name, sub, ctx)
            secondary.append(sec)
        except Exception as exc:  # the headline number must survive a failure of an extra configuration
            secondary.append({"metric": CONFIGS[name][0], "error": f"{type(exc).__name__}: {exc}"[:300]})
    if secondary:
        line["secondary"] = secondary
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        # leave together, and without running the teardown of the communication libraries rank by rank: the result
        # line is out, and nothing below could change it
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)
    return 0


if __name__ == "__main__":
    sys.exit(main())
