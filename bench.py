"""Benchmark of the hot path: dynamic row-wise INT8 quantize + scaled INT8 GEMM (A @ B.T) at 8192^3.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--size S]

One "step" is one pass of the path over one batch of synthetic input:
    weight shard [S/N_gpus, S] bf16 --row-wise quantize--> int8 + scales
        --all-gather over NCCL (N_gpus > 1)--> full int8 weight [S, S] + scales
    activation [S, S] bf16 --row-wise quantize--> int8 + scales
    scaled_mm(int8 A, int8 W^T, row scales, column scales) -> bf16 [S, S]        (tcgen05 kind::i8)
Every rank runs its own activation batch (weak scaling); the weight all-gather is the only exchange.

The line printed by rank 0 follows the driver's contract: whole-job TOPS (`value`), the same
measured through the public API from pinned host buffers (`e2e`), the GEMM's roofline, a CPU
baseline of the same path on the host cores, clocks sampled during the timed region.
`--impl reference` times the reference's CPU form of the path (oracle/cpu_path.py) instead.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "quantized-training_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

METRIC = "scaled_int8_gemm_tops"
UNIT = "TOPS"
NOMINAL_INT8_DENSE_TOPS = 4500.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--size", type=int, default=8192, help="M = N = K")
    ap.add_argument("--mnk", type=int, nargs=3, metavar=("M", "N", "K"), default=None,
                    help="a non-square problem for the gemm workload (profiling the layer shapes; the headline is --size 8192)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-quantize-lines", action="store_true", help="leave the quantize kernels' roofline entries out of the N=1 line")
    ap.add_argument("--workload", default="gemm", choices=["gemm", "quantize", "sweep", "train-470m", "train-1b", "vit-g"],
                    help="gemm: the headline quantize + scaled GEMM step; train-*: one INT8 mixed-precision Llama step (tok/s)")
    ap.add_argument("--parallel", default="fsdp", choices=["ddp", "fsdp"], help="train-* workloads with --gpus > 1: DDP, or FSDP2 with the INT8 weight all-gather")
    ap.add_argument("--quantize", default="mixed_precision", choices=["mixed_precision", "none", "int8_quantized_training", "bitnet"],
                    help="train-* workloads: which weight subclass the decoder's Linear layers get (none = bf16 baseline)")
    ap.add_argument("--gather", default="fused", choices=["fused", "nccl"],
                    help="--gpus > 1: 'fused' = one kernel quantizes the weight shard and stores it into every rank's gathered "
                         "buffer over NVLink (symmetric memory); 'nccl' = quantize, then NCCL all-gather")
    ap.add_argument("--group-m", type=int, default=0, help="force the GEMM's rasterisation group height (0 = the library's choice)")
    ap.add_argument("--sm-margin", type=int, default=None,
                    help="SMs the GEMM leaves free when --gpus > 1 (default: 8 beside NCCL's all-gather kernel, 0 with the fused gather)")
    ap.add_argument("--eager-elementwise", action="store_true",
                    help="train-* workloads: leave RMSNorm, the gated activation and rotary embedding to the model's eager code")
    ap.add_argument("--train-data", default="fixed", choices=["fixed", "markov"],
                    help="train-* workloads: one fixed random batch (throughput), or a fresh batch of learnable synthetic streams per step (loss curves)")
    ap.add_argument("--reduce-fp32", action="store_true", help="train-* workloads with FSDP2: reduce-scatter gradients in fp32")
    ap.add_argument("--no-train-line", action="store_true", help="leave the training throughput measurement out of the default line")
    ap.add_argument("--layers", type=int, default=None, help="train-* workloads: number of decoder layers (default: the model's own)")
    ap.add_argument("--profile", default=None, metavar="FILE",
                    help="train-* workloads: after the timed steps, run two more under torch.profiler and write the kernel table "
                         "(device time per kernel, share of the step) to FILE")
    ap.add_argument("--lead-in-seconds", type=float, default=0.25, help="--workload sweep: untimed replays of a case before it is timed")
    ap.add_argument("--plain-launches", action="store_true", help="--workload quantize: plain launches instead of CUDA-graph replays (for a profiler run)")
    ap.add_argument("--only", default=None, help="--workload quantize: only the kernels whose name contains this text")
    ap.add_argument("--no-triton-comparator", action="store_true", help="--workload sweep: skip the Triton comparator beside the scaled matmuls")
    ap.add_argument("--no-gemm-variants", action="store_true", help="leave the other GEMM forms (FP8, tile-scaled, other layouts) out of the N=1 line")
    ap.add_argument("--no-clock-sampler", action="store_true", help="do not run nvidia-smi beside the timed region")
    ap.add_argument("--min-warmup-seconds", type=float, default=1.0, help="keep warming up at least this long (0 under a profiler)")
    return ap.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        d = json.loads(path.read_text())
        return d.get("hbm_gbs"), d.get("bf16_tflops"), "measured"
    return 6650.0, 1590.0, "fallback"


def measured_sustained_bf16():
    """Dense bf16 TF/s of a seconds-long cuBLAS loop under the power cap (the denominator for a kernel
    timed inside a long loaded step), or the stated fallback."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        v = json.loads(path.read_text()).get("bf16_tflops_sustained")
        if v:
            return float(v), "measured"
    return 1400.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU beside the timed region, through NVML in a
    background thread (the same fields `nvidia-smi --query-gpu=clocks.sm,...` prints; reading only).
    Falls back to an nvidia-smi subprocess when the NVML binding is missing.

    An NVML query can stall the GPU's queued work for milliseconds to tens of milliseconds. The thread
    therefore samples during warm-up only; it is paused around the timed region, and the main thread
    takes the samples that bracket the region itself (see the timed loop) while untimed steps keep the
    GPU under the same load."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, interval_s: float = 0.05):
        self.gpu_index = gpu_index
        self.interval_s = interval_s
        self.samples = []          # (sm_mhz, reasons bitmask)
        self.sm_max = None
        self.thread = None
        self.stop_flag = None
        self.proc = None
        self.file = None
        self.paused = False
        self._read = None

    def pause(self):
        self.paused = True

    def resume(self):
        self.paused = False

    def sample_now(self, n: int = 2):
        """Take n samples on the calling thread (used while the GPU works through queued launches)."""
        if self._read is None:
            return
        for _ in range(n):
            try:
                self.samples.append(self._read())
            except Exception:
                pass

    def start(self):
        try:
            import threading

            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu_index
            if visible:
                try:
                    index = int(visible.split(",")[self.gpu_index])
                except (ValueError, IndexError):
                    index = self.gpu_index
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()

            def read():
                mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                try:
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(handle))
                except Exception:
                    mask = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                return mhz, mask

            self._read = read

            def loop():
                while not self.stop_flag.is_set():
                    if not self.paused:
                        try:
                            self.samples.append(read())
                        except Exception:
                            pass
                    self.stop_flag.wait(self.interval_s)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
        except Exception:
            self.thread = None
            self._start_smi()

    def _start_smi(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "250",
                 "-i", str(self.gpu_index)], stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def mark(self):
        """Samples taken from now on count as 'under load'."""
        self.samples.clear()

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            if self.samples:
                out["sm_mhz"] = statistics.median(m for m, _ in self.samples)
                out["samples"] = len(self.samples)
                mask = 0
                for _, r in self.samples:
                    mask |= r
                out["reasons"] = sorted(name for bit, name in self.REASONS.items() if mask & bit)
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.file.flush()
        self.file.seek(0)
        sm, reasons = [], set()
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                out["sm_max_mhz"] = float(parts[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        if sm:
            out["sm_mhz"] = statistics.median(sm)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def workload_name(M: int, N: int, K: int) -> str:
    """config.workload, spelled the same by both arms."""
    return f"rowwise dynamic INT8 quantize (activation + weight) + scaled INT8 GEMM A@B.T, M={M} N={N} K={K} per GPU, bf16 in/out"


def _bind_near_gpu(gpu_index: int):
    """Run this rank on the CPU cores NVML names as closest to its GPU, so that the pinned host buffers it
    allocates next are first touched, hence placed, on that socket's memory. With eight ranks copying 400 MB
    per step each, buffers on the far socket make every copy cross the inter-socket link. Returns a note for
    the JSON line, or None when the topology cannot be read."""
    try:
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        n_cpu = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        cpus = {64 * w + b for w, mask in enumerate(words) for b in range(64) if (int(mask) >> b) & 1}
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return f"rank bound to the {len(allowed)} CPU cores nearest its GPU before allocating pinned buffers"
    except Exception:   # noqa: BLE001 -- no NVML, no affinity call: stay where we are
        return None


def cpu_reference_step(A, B):
    from oracle import cpu_path

    return cpu_path.dynamic_int8_linear(A, B)


def time_cpu_path(size: int, steps: int, warmup: int):
    """Time the reference's CPU form of the path (torch eager quantize + torch._int_mm + scale) with
    all host threads. Returns (TOPS, threads, seconds per step)."""
    # use every host core (torchrun pins OMP_NUM_THREADS=1 in its workers)
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores))
    torch.manual_seed(2024)
    A = torch.randn(size, size).bfloat16()
    B = (torch.randn(size, size) * 0.02).bfloat16()
    for _ in range(warmup):
        cpu_reference_step(A, B)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference_step(A, B)
    dt = (time.perf_counter() - t0) / steps
    return 2.0 * size ** 3 / dt / 1e12, torch.get_num_threads(), dt


def run_reference(args, rank: int):
    """`--impl reference`: the reference's own CPU implementation of the path, rank 0 only."""
    if rank != 0:
        return
    size = args.size
    # A full 8192^3 pass is seconds of CPU work. The requested warm-up and step counts are honoured as far
    # as a time limit of about two minutes allows: one pass is timed first, and the counts are cut to fit.
    t0 = time.perf_counter()
    time_cpu_path(size, 1, 0)
    one = time.perf_counter() - t0
    passes_that_fit = max(2, int(75.0 / max(one, 1e-3)))
    warmup = max(0, min(args.warmup, passes_that_fit // 4))
    steps = max(1, min(args.steps, passes_that_fit - warmup))
    tops, threads, dt = time_cpu_path(size, steps, warmup)
    sample = (f"{steps} full passes of the {size}^3 workload after {warmup + 1} warm-up passes "
              f"(requested --steps {args.steps} --warmup {args.warmup}; cut to fit 75 s at {one:.1f} s per pass)")
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup + 1, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {"workload": workload_name(size, size, size),
                   "where": "host CPU cores, torch eager quantize + torch._int_mm + scale (oracle/cpu_path.py)"},
        "cpu_baseline": {"value": tops, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


LLAMA_SHAPES = {
    # the reference's shipped config (mini_llamas/Llama-2-470m/config.json:5-10) and the 1.1B shape the reference's README trains (hidden 2048, 22 layers, MLP 5632)
    "train-470m": dict(hidden_size=1024, intermediate_size=4096, num_hidden_layers=24, num_attention_heads=16,
                       num_key_value_heads=16),
    "train-1b": dict(hidden_size=2048, intermediate_size=5632, num_hidden_layers=22, num_attention_heads=32,
                     num_key_value_heads=4),
}


def _markov_tokens(n_seq: int, seq: int, vocab: int, gen: torch.Generator, dev) -> torch.Tensor:
    """Synthetic token streams a model can learn (stand-in for the text corpora the reference trains on, which
    are not available offline): token t+1 = (a * token t + b + noise) mod vocab with a small noise alphabet,
    so the next-token entropy is log(8) instead of log(vocab)."""
    start = torch.randint(0, vocab, (n_seq, 1), generator=gen)
    noise = torch.randint(0, 8, (n_seq, seq), generator=gen)
    out = torch.empty((n_seq, seq + 1), dtype=torch.long)
    out[:, :1] = start
    for t in range(seq):
        out[:, t + 1] = (out[:, t] * 31 + 7 + noise[:, t]) % vocab
    return out.to(dev)


def train_measure(workload: str, quantize: str, parallel: str, steps: int, warmup: int, rank: int, local_rank: int, world: int, *,
                  layers=None, eager_elementwise=False, data="fixed", profile=None, reduce_fp32=False) -> dict:
    """One measurement of the training workload (the process group, if any, is already up): returns the fields of
    the JSON line. INT8 mixed-precision training step of a random-init Llama-style decoder (forward, grad-input
    and grad-weight GEMMs all row-wise INT8; LM head in bf16; AdamWBF16SR), batch 16 x 2048 tokens per GPU,
    tok/s as the reference computes it (llm_pretrain.py:229-234). With several ranks: FSDP2 per decoder layer
    (llm_pretrain.py:134-139) with the INT8 weight all-gather, or DDP."""
    from transformers import LlamaConfig, LlamaForCausalLM

    from train_utils import fuse_decoder_elementwise, get_optimizer, quantize_model

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    bs, seq = 16, 2048
    torch.manual_seed(2024)
    shape = dict(LLAMA_SHAPES[workload])
    if layers is not None:
        shape["num_hidden_layers"] = layers
    cfg = LlamaConfig(vocab_size=32000, max_position_embeddings=seq, attn_implementation="sdpa", tie_word_embeddings=False, **shape)
    with torch.device(dev):
        model = LlamaForCausalLM(cfg).bfloat16()
    quantize_model(model.model, None if quantize == "none" else quantize)
    if not eager_elementwise:
        # RMSNorm / silu * up / rotary embedding as single kernels; they emit the int8 activations where INT8 linears follow
        fuse_decoder_elementwise(model)
    if world > 1 and parallel == "fsdp":
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

        kw = {"mp_policy": MixedPrecisionPolicy(reduce_dtype=torch.float32)} if reduce_fp32 else {}
        for layer in model.model.layers:   # per decoder layer, then the root (llm_pretrain.py:134-139)
            fully_shard(layer, **kw)
        fully_shard(model, **kw)
    elif world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])
    optim = get_optimizer("other_optim.AdamWBF16SR", model, lr=1e-4 if data == "fixed" else 3e-4, weight_decay=0.01)
    gen = torch.Generator().manual_seed(2024 + rank)
    fixed = torch.randint(0, 32000, (bs, seq + 1), generator=gen).to(dev)
    losses = []

    def step():
        tokens = fixed if data == "fixed" else _markov_tokens(bs, seq, 1024, gen, dev)   # a 1024-token alphabet of the 32000
        logits = model(input_ids=tokens[:, :-1]).logits.float()
        loss = torch.nn.functional.cross_entropy(logits.view(-1, logits.shape[-1]), tokens[:, 1:].reshape(-1))
        loss.backward()
        optim.step()
        optim.zero_grad(set_to_none=True)
        losses.append(loss.detach())
        return loss

    warmup = max(warmup, 3)
    for _ in range(warmup):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    if profile and rank == 0 and world == 1:
        from torch.profiler import ProfilerActivity
        from torch.profiler import profile as torch_profile

        with torch_profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA]) as prof:
            for _ in range(2):
                step()
            torch.cuda.synchronize()
        rows = [(k.key, k.count, getattr(k, "device_time_total", getattr(k, "cuda_time_total", 0.0)))
                for k in prof.key_averages() if getattr(k, "device_type", None) is not None and "cuda" in str(k.device_type).lower()]
        total = sum(r[2] for r in rows) or 1.0
        rows.sort(key=lambda r: -r[2])
        with open(profile, "w") as f:
            f.write(f"# {workload} layers={shape['num_hidden_layers']} quantize={quantize}: device time per kernel over 2 steps "
                    f"(torch.profiler); step {ms / steps:.2f} ms by CUDA events, kernels sum to {total / 2e3:.2f} ms per step\n")
            f.write("share%  total_us  launches  kernel\n")
            for name, count, us in rows[:60]:
                f.write(f"{100 * us / total:6.2f} {us:9.0f} {count:9d}  {name[:150]}\n")
    n_params = sum(p.numel() for p in model.parameters())
    out = {
        "metric": "int8_mixed_precision_train_tok_per_s", "value": world * bs * seq * steps / (ms * 1e-3), "unit": "tok/s",
        "n_gpus": world, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8" if quantize != "none" else "bf16", "data": "synthetic",
        "config": {"workload": f"{workload}: Llama-style decoder, {n_params / 1e6:.0f}M params, {shape['num_hidden_layers']} layers, quantize={quantize} "
                               f"(LM head bf16), AdamWBF16SR, batch {bs} x {seq} tokens per GPU "
                               f"({'one fixed random batch' if data == 'fixed' else 'a fresh batch of learnable synthetic streams per step'}), "
                               f"{'eager' if eager_elementwise else 'fused'} element-wise kernels",
                   "parallelism": (f"fsdp{world}" + (" fp32 reduce-scatter" if reduce_fp32 else "") if (world > 1 and parallel == "fsdp") else f"dp{world}")},
        "loss": float(loss.detach()), "losses": [round(float(x), 4) for x in losses], "max_memory_gb": torch.cuda.max_memory_allocated() / 1e9,
    }
    del model, optim
    gc.collect()
    torch.cuda.empty_cache()
    return out


def run_train(args, rank, local_rank, world):
    """`--workload train-*`: see train_measure."""
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    line = train_measure(args.workload, args.quantize, args.parallel, args.steps, args.warmup, rank, local_rank, world, layers=args.layers,
                         eager_elementwise=args.eager_elementwise, data=args.train_data, profile=args.profile, reduce_fp32=args.reduce_fp32)
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


VIT_G14 = dict(dim=1536, depth=40, heads=24, mlp=6144, image=224, patch=14, classes=45)


def _build_vit(cfg: dict, dev):
    """ViT-giant/14 as the reference fine-tunes it (timm_finetune.py:136-139 creates timm's
    vit_giant_patch14_224 with 45 classes): patch embedding, class token, learned positions, pre-norm blocks
    (LayerNorm, fused-QKV attention, GELU MLP), final norm, linear head. Random init: the pretrained
    checkpoint and the dataset are not available offline."""
    nn = torch.nn

    class Block(nn.Module):
        def __init__(self, dim, heads, mlp):
            super().__init__()
            self.norm1, self.norm2 = nn.LayerNorm(dim, eps=1e-6), nn.LayerNorm(dim, eps=1e-6)
            self.qkv, self.proj = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
            self.fc1, self.fc2 = nn.Linear(dim, mlp), nn.Linear(mlp, dim)
            self.heads = heads

        def forward(self, x):
            b, n, d = x.shape
            qkv = self.qkv(self.norm1(x)).view(b, n, 3, self.heads, d // self.heads).permute(2, 0, 3, 1, 4)
            a = torch.nn.functional.scaled_dot_product_attention(qkv[0], qkv[1], qkv[2])
            x = x + self.proj(a.transpose(1, 2).reshape(b, n, d))
            return x + self.fc2(torch.nn.functional.gelu(self.fc1(self.norm2(x))))

    class ViT(nn.Module):
        def __init__(self, dim, depth, heads, mlp, image, patch, classes):
            super().__init__()
            self.patch = patch
            n = (image // patch) ** 2
            self.embed = nn.Linear(3 * patch * patch, dim)
            self.cls = nn.Parameter(torch.zeros(1, 1, dim))
            self.pos = nn.Parameter(torch.randn(1, n + 1, dim) * 0.02)
            self.blocks = nn.ModuleList(Block(dim, heads, mlp) for _ in range(depth))
            self.norm = nn.LayerNorm(dim, eps=1e-6)
            self.head = nn.Linear(dim, classes)

        def forward(self, img):
            b, c, h, w = img.shape
            p = self.patch
            x = img.view(b, c, h // p, p, w // p, p).permute(0, 2, 4, 1, 3, 5).reshape(b, (h // p) * (w // p), c * p * p)
            x = torch.cat((self.cls.expand(b, -1, -1), self.embed(x)), dim=1) + self.pos
            for blk in self.blocks:
                x = blk(x)
            return self.head(self.norm(x)[:, 0])

    with torch.device(dev):
        return ViT(**cfg).bfloat16()


def run_vit(args, rank, local_rank, world):
    """`--workload vit-g`: one training step of ViT-giant/14 (dim 1536, 40 layers, 24 heads, MLP 6144, 224x224,
    patch 14, 45 classes), batch 64 random images per GPU, with the INT8 weight-only subclass
    (int8 row-scaled weights, stochastic-rounding update; --quantize int8_quantized_training), the BitNet b1.58
    variant (--quantize bitnet) or bf16 (--quantize none); DDP over the ranks. Images per second."""
    from train_utils import quantize_model

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    cfg = dict(VIT_G14)
    if args.layers is not None:
        cfg["depth"] = args.layers
    torch.manual_seed(2024)
    model = _build_vit(cfg, dev)
    quantize = None if args.quantize == "none" else args.quantize
    quantize_model(model.blocks, quantize)      # the transformer blocks; patch embedding and head stay bf16
    n_params = sum(p.numel() for p in model.parameters())
    if world > 1:
        model = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])
    optim = torch.optim.AdamW(model.parameters(), lr=1e-5, weight_decay=0.01)
    bs = 64
    gen = torch.Generator().manual_seed(2024 + rank)
    images = torch.randn(bs, 3, cfg["image"], cfg["image"], generator=gen).bfloat16().to(dev)
    labels = torch.randint(0, cfg["classes"], (bs,), generator=gen).to(dev)

    def step():
        loss = torch.nn.functional.cross_entropy(model(images).float(), labels)
        loss.backward()
        optim.step()
        optim.zero_grad(set_to_none=True)
        return loss

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        print(json.dumps({
            "metric": "vit_train_images_per_s", "value": world * bs * args.steps / (ms * 1e-3), "unit": "img/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8" if quantize else "bf16", "data": "synthetic",
            "config": {"workload": f"ViT-giant/14, {n_params / 1e6:.0f}M params, {cfg['depth']} layers, quantize={args.quantize}, torch AdamW, "
                                   f"batch {bs} x 3 x {cfg['image']} x {cfg['image']} random images per GPU, random labels",
                       "parallelism": f"dp{world}"},
            "loss": float(loss.detach()), "max_memory_gb": torch.cuda.max_memory_allocated() / 1e9}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _time_graph(launch, n_sets: int, launches: int, reps: int = 5, graph: bool = True, lead_in_s: float = 0.0) -> float:
    """Milliseconds per launch of `launch(i)` (i = which buffer set), measured over a CUDA graph of
    `launches` back-to-back launches that rotate through `n_sets` buffer sets. The sets together are several
    times larger than L2, so every launch reads its input from HBM and the dirty lines it displaces are a
    previous launch's output of the same kernel: steady-state traffic equals the algorithmic bytes. Events
    bracket whole graph replays (no host launch gaps, no event overhead per launch); the median replay counts."""
    for i in range(n_sets):
        launch(i)
    torch.cuda.synchronize()
    if not graph:   # plain launches between two events (what a profiler run uses): host launch gaps included
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(launches):
            launch(i % n_sets)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / launches
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(launches):
            launch(i % n_sets)
    g.replay()
    torch.cuda.synchronize()
    if lead_in_s > 0.0:
        # untimed replays first, so that every case is timed in the same loaded (power-capped) state instead of
        # whatever state the previous case left behind
        t0 = time.perf_counter()
        while time.perf_counter() - t0 < lead_in_s:
            for _ in range(4):
                g.replay()
            torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / launches)
    return statistics.median(times)


def quantize_lines(M: int, K: int, launches: int, dev, graph: bool = True, only: str | None = None) -> list:
    """Roofline entries for the HBM-bound kernels of the path on [M, K] bf16 (N(0,1)) through the C ABI with
    preallocated outputs: algorithmic bytes, time per launch (_time_graph) and the fraction of the measured
    HBM copy bandwidth."""
    from gn_kernels import _native as nv

    lib = nv.load()
    hbm_peak, _, peak_kind = measured_peaks()
    RC = M * K
    n_sets = max(3, -(-3 * 126 * (1 << 20) // (3 * RC)) + 1)
    xs = [torch.randn(M, K, device=dev).bfloat16() for _ in range(n_sets)]
    qs = [torch.empty(M, K, dtype=torch.int8, device=dev) for _ in range(n_sets)]
    qts = [torch.empty(K, M, dtype=torch.int8, device=dev) for _ in range(n_sets)]
    row_scales = [torch.empty(M, 1, dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    col_scales = [torch.empty(K, 1, dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    tile_scales = [torch.empty(M, -(-K // 128), dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    colmaxes = [torch.empty(K, dtype=torch.float32, device=dev) for _ in range(n_sets)]
    BF16, I8, E4M3 = nv.QT_BF16, nv.QT_I8, nv.QT_E4M3

    def st():
        return nv.stream_ptr(dev)

    def rowwise(q_dtype, sr):
        def f(i):
            nv.check(lib.qt_quantize_rowwise(xs[i].data_ptr(), BF16, M, K, K, qs[i].data_ptr(), q_dtype, row_scales[i].data_ptr(),
                                             BF16, 1e-12, int(sr), 2024, 1 + i, st()))
        return f

    def rowwise_colabs(i):
        nv.check(lib.qt_quantize_rowwise_colabsmax(xs[i].data_ptr(), BF16, M, K, K, qs[i].data_ptr(), I8, row_scales[i].data_ptr(), BF16,
                                                   colmaxes[i].data_ptr(), 1e-12, 0, 0, 0, st()))

    def col_absmax(i):
        nv.check(lib.qt_col_absmax(xs[i].data_ptr(), BF16, M, K, K, colmaxes[i].data_ptr(), st()))

    def colwise_t(i):
        nv.check(lib.qt_quantize_colwise_t(xs[i].data_ptr(), BF16, M, K, K, colmaxes[i].data_ptr(), qts[i].data_ptr(), I8,
                                           col_scales[i].data_ptr(), BF16, 1e-12, 0, 0, 0, st()))

    def tile(tr, q_dtype):
        def f(i):
            nv.check(lib.qt_quantize_tile(xs[i].data_ptr(), BF16, M, K, K, tr, 128, qs[i].data_ptr(), q_dtype, tile_scales[i].data_ptr(),
                                          BF16, 1e-12, st()))
        return f

    # the INT8 weight-only optimizer step on an [M, K] int8 weight: read q, t1, t2 and write q (6 B / weight)
    t1s = [torch.randn(M, K, device=dev).bfloat16() * 1e-3 for _ in range(n_sets)]

    def weight_update(i):
        nv.check(lib.qt_int8_weight_update(qs[i].data_ptr(), row_scales[i].data_ptr(), M, K, 1, t1s[i].data_ptr(), xs[i].data_ptr(),
                                           -1e-3, 1e-12, 2024, 1 + i, st()))

    # multi-tensor AdamW with bf16 stochastic rounding on 8 tensors of RC / 8 elements (p, g, m, v all bf16: 14 B / parameter)
    import ctypes

    n_t, per = 8, RC // 8
    ptr_t, len_t = ctypes.c_void_p * n_t, ctypes.c_int64 * n_t
    ms_ = [torch.zeros(M, K, dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    vs_ = [torch.zeros(M, K, dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    ps_ = [torch.randn(M, K, device=dev).bfloat16() for _ in range(n_sets)]

    def adamw_multi(i):
        def tab(t):
            return ptr_t(*[t.data_ptr() + 2 * per * j for j in range(n_t)])
        nv.check(lib.qt_adamw_bf16_sr_multi(n_t, tab(ps_[i]), tab(xs[i]), tab(ms_[i]), tab(vs_[i]), len_t(*[per] * n_t), BF16, BF16,
                                            1e-4, 0.9, 0.999, 0.01, 1e-8, 0.1, 0.0316, 1, 2024, 1 + 8 * i, st()))

    # BitNet weight ternarisation (2-bit packed): read bf16, write a quarter byte per weight
    bscale = torch.full((1,), 0.8, dtype=torch.float32, device=dev)
    packed = [torch.empty(RC // 4, dtype=torch.int8, device=dev) for _ in range(n_sets)]

    def ternary(i):
        nv.check(lib.qt_bitnet_quantize_weight(xs[i].data_ptr(), BF16, RC, bscale.data_ptr(), 1e-5, packed[i].data_ptr(), 1, st()))

    for i in range(n_sets):   # the column-wise kernel and the weight update read what these write
        col_absmax(i)
        rowwise(I8, False)(i)
    cases = [
        ("rowwise_full_kernel int8", rowwise(I8, False), 3 * RC + 2 * M),
        ("rowwise_full_kernel int8 stochastic", rowwise(I8, True), 3 * RC + 2 * M),
        ("rowwise_full_kernel e4m3", rowwise(E4M3, False), 3 * RC + 2 * M),
        ("rowwise_full_kernel int8 + column absmax", rowwise_colabs, 3 * RC + 2 * M + 4 * K),
        ("col_absmax_bf16_kernel", col_absmax, 2 * RC + 4 * K),
        ("colwise_t_fast_kernel int8 (given column absmax)", colwise_t, 3 * RC + 6 * K),
        ("rowwise_full_kernel<TILE> 1x128 int8", tile(1, I8), 3 * RC + 2 * RC // 128),
        ("rowwise_full_kernel<TILE> 1x128 e4m3", tile(1, E4M3), 3 * RC + 2 * RC // 128),
        ("tile_128x128_fast_kernel int8", tile(128, I8), 3 * RC + 2 * RC // 16384),
        ("rowwise_kernel<UPD> int8 weight update (addcdiv, stochastic)", weight_update, 6 * RC + 4 * M),
        ("adamw_multi_kernel bf16 stochastic", adamw_multi, 14 * RC),
        ("ternary_kernel 2-bit packed", ternary, 2 * RC + RC // 4),
    ]
    out = []
    for name, fn, nbytes in cases:
        if only and only not in name:
            continue
        ms = _time_graph(fn, n_sets, launches, graph=graph)
        gbs = nbytes / (ms * 1e-3) / 1e9
        out.append({"kernel": name, "us_per_launch": round(ms * 1e3, 2), "algorithmic_bytes": nbytes, "achieved": round(gbs, 1),
                    "peak": hbm_peak, "unit": "GB/s", "frac": round(gbs / hbm_peak, 3), "frac_of_nominal_8tbs": round(gbs / 8000.0, 3),
                    "bound": "hbm", "peak_is": f"{peak_kind} STREAM-style copy"})
    out.append({"shape": [M, K], "launches_per_graph": launches, "buffer_sets": n_sets,
                "l2": "launches rotate through buffer sets several times larger than L2; timed as CUDA-graph replays"})
    return out


_TRITON_COMPARATOR = None


def _triton_scaled_mm_comparator():
    """A Triton row/column-scaled INT8 / FP8 matmul of the usual tiled form (program per output tile, grouped
    rasterisation, K loop of tl.dot, scales applied to the accumulator in the epilogue) -- the structure of the
    kernel the reference runs (kernels/gn_kernels/triton_mm.py:146-220), written here from that description.
    A comparator for the sweep only: nothing in the product imports Triton. Returns fn(A, B, sa, sb) -> bf16
    [M, N] that tries a few tile shapes on first use and keeps the fastest, or None when Triton is unusable."""
    global _TRITON_COMPARATOR
    if _TRITON_COMPARATOR is not None:
        return _TRITON_COMPARATOR or None
    try:
        import triton
        import triton.language as tl
    except Exception:   # noqa: BLE001
        _TRITON_COMPARATOR = False
        return None

    @triton.jit
    def kernel(a_ptr, b_ptr, c_ptr, sa_ptr, sb_ptr, M, N, K, sam, sak, sbk, sbn, scm, scn,
               BM: tl.constexpr, BN: tl.constexpr, BK: tl.constexpr, GROUP_M: tl.constexpr, INT8: tl.constexpr):
        pid = tl.program_id(0)
        tiles_m = tl.cdiv(M, BM)
        tiles_n = tl.cdiv(N, BN)
        width = GROUP_M * tiles_n
        group = pid // width
        first_m = group * GROUP_M
        group_size = min(tiles_m - first_m, GROUP_M)
        pid_m = first_m + (pid % width) % group_size
        pid_n = (pid % width) // group_size
        offs_m = pid_m * BM + tl.arange(0, BM)
        offs_n = pid_n * BN + tl.arange(0, BN)
        offs_k = tl.arange(0, BK)
        a_ptrs = a_ptr + offs_m[:, None] * sam + offs_k[None, :] * sak
        b_ptrs = b_ptr + offs_k[:, None] * sbk + offs_n[None, :] * sbn
        if INT8:
            acc = tl.zeros((BM, BN), dtype=tl.int32)
        else:
            acc = tl.zeros((BM, BN), dtype=tl.float32)
        for _ in range(0, tl.cdiv(K, BK)):   # the sweep's sizes are multiples of every tile shape tried
            a = tl.load(a_ptrs)
            b = tl.load(b_ptrs)
            if INT8:
                acc = tl.dot(a, b, acc, out_dtype=tl.int32)
            else:
                acc = tl.dot(a, b, acc)
            a_ptrs += BK * sak
            b_ptrs += BK * sbk
        sa = tl.load(sa_ptr + offs_m).to(tl.float32)
        sb = tl.load(sb_ptr + offs_n).to(tl.float32)
        out = acc.to(tl.float32) * sa[:, None] * sb[None, :]
        tl.store(c_ptr + offs_m[:, None] * scm + offs_n[None, :] * scn, out.to(tl.bfloat16))

    configs = [(128, 256, 128, 3, 8), (128, 128, 128, 4, 4), (256, 128, 128, 3, 8), (128, 256, 64, 4, 8), (128, 128, 64, 4, 4)]
    best = {}

    def run(A, B, sa, sb, cfg=None):
        M, K = A.shape
        N = B.shape[1]
        key = (M, N, K, A.dtype, A.stride(), B.stride())
        C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)

        def launch(c):
            bm, bn, bk, stages, warps = c
            grid = (triton.cdiv(M, bm) * triton.cdiv(N, bn),)
            kernel[grid](A, B, C, sa, sb, M, N, K, A.stride(0), A.stride(1), B.stride(0), B.stride(1), C.stride(0), C.stride(1),
                         BM=bm, BN=bn, BK=bk, GROUP_M=8, INT8=(A.dtype == torch.int8), num_stages=stages, num_warps=warps)

        if key not in best:
            timed, why = [], "no tile shape divides the problem"
            for c in configs:
                if M % c[0] or N % c[1] or K % c[2]:
                    continue
                try:
                    launch(c)
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(5):
                        launch(c)
                    e1.record()
                    torch.cuda.synchronize()
                    timed.append((e0.elapsed_time(e1), c))
                except Exception as exc:   # noqa: BLE001 -- a tile shape this Triton cannot compile or fit
                    why = f"{type(exc).__name__}: {str(exc)[-300:]}"
                    continue
            if not timed:
                raise RuntimeError(f"no Triton tile shape compiled ({why})")
            best[key] = min(timed)[1]
        launch(best[key])
        return C

    run.best = best
    _TRITON_COMPARATOR = run
    return run


def run_sweep(args):
    """The reference's GEMM benchmark grid (benchmark_mm.py:33-34,70-145): M = N = K in {1024, 2048, 4096, 8192}
    x layouts {A@B.T, A@B, A.T@B} x {int8_mm, row-scaled INT8, row-scaled FP8 e4m3, tile-scaled INT8, tile-scaled
    FP8}; 2*M*N*K / time (benchmark_mm.py:107). One JSON line per cell with the library GEMM of the same box
    beside it where one exists (torch._int_mm; torch._scaled_mm with row-wise scales, A@B.T only). Operands are
    random int8 / e4m3 values with random bf16 scales (timing only; parity is the tests' job). Launches rotate
    through operand sets several times larger than L2 and are timed as CUDA-graph replays (_time_graph)."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    import gn_kernels

    dev = torch.device("cuda", 0)
    _, bf16_peak, peak_kind = measured_peaks()
    peak = 2.0 * bf16_peak
    sizes = [args.size] if args.size != 8192 or args.only else [1024, 2048, 4096, 8192]
    if args.only and args.only.isdigit():
        sizes = [int(args.only)]
    launches = max(args.steps, 10)

    def layout(t, col_major):
        return t.T.contiguous().T if col_major else t.contiguous()

    for S in sizes:
        M = N = K = S
        per_launch = 2 * S * S + 2 * S * S          # int8 operands + bf16 result
        n_sets = min(48, max(3, -(-3 * 126 * (1 << 20) // per_launch) + 1))
        for lname, a_col, b_col in (("A@B.T", False, True), ("A@B", False, False), ("A.T@B", True, False)):
            A8 = [layout(torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev), a_col) for _ in range(n_sets)]
            B8 = [layout(torch.randint(-128, 128, (K, N), dtype=torch.int8, device=dev), b_col) for _ in range(n_sets)]
            Af = [t.to(torch.bfloat16).mul_(0.01).to(torch.float8_e4m3fn) for t in A8]
            Bf = [t.to(torch.bfloat16).mul_(0.01).to(torch.float8_e4m3fn) for t in B8]
            Af = [layout(t, a_col) for t in Af]
            Bf = [layout(t, b_col) for t in Bf]
            sa = (torch.rand(M, 1, device=dev) * 0.01 + 0.001).bfloat16()
            sb = (torch.rand(1, N, device=dev) * 0.01 + 0.001).bfloat16()
            ta = (torch.rand(M, K // 128, device=dev) * 0.01 + 0.001).bfloat16()
            tb = (torch.rand(K // 128, N // 128, device=dev) * 0.01 + 0.001).bfloat16()
            cases = [
                ("int8_mm", lambda i: gn_kernels.int8_mm(A8[i], B8[i]), lambda i: torch._int_mm(A8[i], B8[i]), "torch._int_mm"),
                ("scaled_mm int8", lambda i: gn_kernels.scaled_mm(A8[i], B8[i], sa, sb),
                 lambda i: (torch._int_mm(A8[i], B8[i]).float().mul_(sa.float()).mul_(sb.float())).bfloat16(), "torch._int_mm + eager scaling"),
                ("scaled_mm e4m3", lambda i: gn_kernels.scaled_mm(Af[i], Bf[i], sa, sb),
                 (lambda i: torch._scaled_mm(Af[i], Bf[i], scale_a=sa.float(), scale_b=sb.float(), out_dtype=torch.bfloat16))
                 if (not a_col and b_col) else None, "torch._scaled_mm row-wise"),
                ("tile_scaled_mm int8 (1x128, 128x128)", lambda i: gn_kernels.scaled_mm(A8[i], B8[i], ta, tb), None, None),
                ("tile_scaled_mm e4m3 (1x128, 128x128)", lambda i: gn_kernels.scaled_mm(Af[i], Bf[i], ta, tb), None, None),
            ]
            for name, fn, lib_fn, lib_name in cases:
                if args.only and not args.only.isdigit() and args.only not in name:
                    continue
                ms = _time_graph(fn, n_sets, launches, lead_in_s=args.lead_in_seconds)
                tops = 2.0 * M * N * K / (ms * 1e-3) / 1e12
                line = {"metric": "gemm_tops", "kernel": name, "layout": lname, "size": S, "value": round(tops, 1), "unit": "TOPS",
                        "us_per_launch": round(ms * 1e3, 2), "frac_of_2x_measured_bf16": round(tops / peak, 3),
                        "frac_of_nominal_4500": round(tops / NOMINAL_INT8_DENSE_TOPS, 3), "peak": peak, "peak_is": f"2 x {peak_kind} dense bf16 burst",
                        "n_gpus": 1, "steps": launches, "higher_is_better": True, "data": "synthetic",
                        "config": {"workload": f"{name} {lname} M=N=K={S}", "l2": f"{n_sets} operand sets in rotation, CUDA-graph replays",
                                   "lead_in_seconds": args.lead_in_seconds}}
                if lib_fn is not None:
                    try:
                        lms = _time_graph(lib_fn, n_sets, launches, lead_in_s=args.lead_in_seconds)
                        line["library"] = {"what": lib_name, "tops": round(2.0 * M * N * K / (lms * 1e-3) / 1e12, 1), "us_per_launch": round(lms * 1e3, 2)}
                    except Exception as exc:   # a layout or shape the library refuses
                        line["library"] = {"what": lib_name, "unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}
                if name.startswith("scaled_mm") and not args.no_triton_comparator:
                    tri = _triton_scaled_mm_comparator()
                    ops = (A8, B8) if "int8" in name else (Af, Bf)
                    if tri is None:
                        line["triton_comparator"] = {"unavailable": "import triton failed"}
                    else:
                        try:
                            tms = _time_graph(lambda i: tri(ops[0][i], ops[1][i], sa, sb), n_sets, launches, lead_in_s=args.lead_in_seconds)
                            cfg = tri.best.get((M, N, K, ops[0][0].dtype, ops[0][0].stride(), ops[1][0].stride()))
                            line["triton_comparator"] = {"what": "own Triton restatement of the reference's scaled matmul (comparator only)",
                                                         "tops": round(2.0 * M * N * K / (tms * 1e-3) / 1e12, 1), "us_per_launch": round(tms * 1e3, 2),
                                                         "tile_stages_warps": list(cfg) if cfg else None}
                        except Exception as exc:   # noqa: BLE001
                            line["triton_comparator"] = {"unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}
                print(json.dumps(line), flush=True)
            del A8, B8, Af, Bf
            torch.cuda.empty_cache()


def gemm_variant_lines(dev, size: int = 8192, launches: int = 10, lead_in_s: float = 0.15) -> list:
    """The other GEMM forms of the path at size^3, for the default line: raw INT8, row-scaled INT8 in the two other
    layouts, row-scaled FP8, tile-scaled INT8 and FP8 (A@B.T unless the name says otherwise). Same timing as the
    sweep (CUDA-graph replays over rotating operand sets, a short loaded lead-in); fractions against twice the
    measured bf16 burst and against the nominal dense rate."""
    import gn_kernels

    _, bf16_peak, peak_kind = measured_peaks()
    peak = 2.0 * bf16_peak
    S = size
    n_sets = 3

    def col(t):
        return t.T.contiguous().T

    A8 = [torch.randint(-128, 128, (S, S), dtype=torch.int8, device=dev) for _ in range(n_sets)]
    B8 = [torch.randint(-128, 128, (S, S), dtype=torch.int8, device=dev) for _ in range(n_sets)]
    sa = (torch.rand(S, 1, device=dev) * 0.01 + 0.001).bfloat16()
    sb = (torch.rand(1, S, device=dev) * 0.01 + 0.001).bfloat16()
    ta = (torch.rand(S, S // 128, device=dev) * 0.01 + 0.001).bfloat16()
    tb = (torch.rand(S // 128, S // 128, device=dev) * 0.01 + 0.001).bfloat16()
    out = []

    def add(name, fn):
        try:
            ms = _time_graph(fn, n_sets, launches, lead_in_s=lead_in_s)
            tops = 2.0 * S ** 3 / (ms * 1e-3) / 1e12
            out.append({"kernel": name, "size": S, "tops": round(tops, 1), "us_per_launch": round(ms * 1e3, 1),
                        "frac_of_2x_measured_bf16": round(tops / peak, 3), "frac_of_nominal_4500": round(tops / NOMINAL_INT8_DENSE_TOPS, 3)})
        except Exception as exc:   # noqa: BLE001 -- a missing entry must not lose the line
            out.append({"kernel": name, "size": S, "error": f"{type(exc).__name__}: {str(exc)[:160]}"})

    Bt = [col(b) for b in B8]                                    # [K, N] with K contiguous: A@B.T
    add("int8_mm A@B.T (int32 out)", lambda i: gn_kernels.int8_mm(A8[i], Bt[i]))
    add("scaled_mm int8 A@B", lambda i: gn_kernels.scaled_mm(A8[i], B8[i], sa, sb))
    At = [col(a) for a in A8]
    add("scaled_mm int8 A.T@B", lambda i: gn_kernels.scaled_mm(At[i], B8[i], sa, sb))
    del At
    add("tile_scaled_mm int8 (1x128, 128x128) A@B.T", lambda i: gn_kernels.scaled_mm(A8[i], Bt[i], ta, tb))
    Af = [a.to(torch.bfloat16).mul_(0.01).to(torch.float8_e4m3fn) for a in A8]
    Bf = [col(b.to(torch.bfloat16).mul_(0.01).to(torch.float8_e4m3fn)) for b in B8]
    del A8, B8, Bt
    add("scaled_mm e4m3 A@B.T", lambda i: gn_kernels.scaled_mm(Af[i], Bf[i], sa, sb))
    add("tile_scaled_mm e4m3 (1x128, 128x128) A@B.T", lambda i: gn_kernels.scaled_mm(Af[i], Bf[i], ta, tb))
    out.append({"timed_as": f"CUDA-graph replays of {launches} launches over {n_sets} operand sets, {lead_in_s} s loaded lead-in, median of 5",
                "peak": peak, "peak_is": f"2 x {peak_kind} dense bf16 burst"})
    return out


def run_quantize(args):
    """The HBM-bound kernels of the path on one [M, K] bf16 tensor (--mnk M N K; N is ignored; default
    32768 x 2048, the activation of a 2048-wide layer at 32768 tokens): one JSON line per kernel."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    dev = torch.device("cuda", 0)
    M, _, K = tuple(args.mnk) if args.mnk else (32768, 0, 2048)
    lines = quantize_lines(M, K, max(args.steps, 2), dev, graph=not args.plain_launches, only=args.only)
    how = lines[-1]
    for e in lines[:-1]:
        print(json.dumps({"metric": "quantize_gbs", "kernel": e["kernel"], "value": e["achieved"], "unit": "GB/s", "n_gpus": 1,
                          "steps": how["launches_per_graph"], "ms_per_launch": e["us_per_launch"] / 1e3, "higher_is_better": True,
                          "dtype": "bf16->int8/fp8", "data": "synthetic",
                          "config": {"workload": f"[{M}, {K}] bf16 N(0,1)", "l2": how["l2"], "buffer_sets": how["buffer_sets"]},
                          "roofline": {k: e[k] for k in ("bound", "achieved", "peak", "unit", "frac", "frac_of_nominal_8tbs", "peak_is", "algorithmic_bytes")}}),
              flush=True)


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "quantize":
        if rank == 0:
            run_quantize(args)
        return
    if args.workload == "sweep":
        if rank == 0:
            run_sweep(args)
        return
    if args.workload == "vit-g":
        run_vit(args, rank, local_rank, world)
        return
    if args.workload != "gemm":
        run_train(args, rank, local_rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback (use --impl reference for the CPU arm)")

    import gn_kernels
    from gn_kernels import _native

    _native.load()
    if args.group_m:
        _native.check(_native.load().qt_set_gemm_group_m(args.group_m))
    fused_gather = world > 1 and args.gather == "fused"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    numa_note = _bind_near_gpu(local_rank) if world > 1 else None
    S = args.size
    gM, gN, gK = tuple(args.mnk) if args.mnk else (S, S, S)
    assert gN % world == 0, "the weight rows must split evenly over the ranks"
    shard_rows = gN // world
    torch.manual_seed(2024 + rank)
    A_host = torch.randn(gM, gK).bfloat16().pin_memory()
    torch.manual_seed(2024)  # the weight is the same tensor on every rank; each rank owns a row slice
    W_full_host = (torch.randn(gN, gK) * 0.02).bfloat16()
    W_host = W_full_host[rank * shard_rows:(rank + 1) * shard_rows].contiguous().pin_memory()
    del W_full_host
    A = A_host.to(dev)
    W = W_host.to(dev)
    out_host = torch.empty((gM, gN), dtype=torch.bfloat16).pin_memory()

    # Gathered weight, double-buffered: with more than one GPU the quantize + all-gather of the NEXT
    # step's weight runs on a side stream under the current step's activation quantize and GEMM (the
    # prefetch FSDP2 does for the next layer), so every step still holds exactly one shard quantize,
    # one all-gather, one activation quantize and one GEMM.
    sym, gather_note = None, None
    if fused_gather:
        # every rank must take the same path: agree on whether the symmetric buffers could be set up
        try:
            from gn_kernels.sharded import SymmetricRowGather
            sym = SymmetricRowGather(gN, gK, device=dev, buffers=3)
            ok_here = 1
        except Exception as exc:  # no symmetric memory on this system: the NCCL all-gather serves
            gather_note = f"fused gather unavailable ({type(exc).__name__}: {exc}); NCCL all-gather used"
            ok_here = 0
        agree = torch.tensor([ok_here], dtype=torch.int32, device=dev)
        dist.all_reduce(agree, op=dist.ReduceOp.MIN)
        if int(agree.item()) == 0:
            sym, fused_gather = None, False
            gather_note = gather_note or "fused gather unavailable on another rank; NCCL all-gather used"
    if args.sm_margin is None:
        # NCCL's all-gather kernels need SMs beside the persistent GEMM; the fused form only has its 4-byte
        # fence (one CTA) and the first CTAs of the scatter kernel to place while a GEMM is running
        args.sm_margin = 0 if world == 1 else (2 if fused_gather else 8)
    if world > 1:
        _native.check(_native.load().qt_set_gemm_sm_margin(args.sm_margin))
    if sym is not None:
        wq_full, ws_full = sym.q, sym.scale
    else:
        wq_full = [torch.empty((gN, gK), dtype=torch.int8, device=dev) for _ in range(2)]
        ws_full = [torch.empty((gN, 1), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    comm_stream = torch.cuda.Stream(device=dev) if world > 1 else None
    n_wbuf = len(wq_full)                                    # 2 with NCCL, 3 with the fused gather
    gathered = [torch.cuda.Event() for _ in range(n_wbuf)]   # buffer b holds a complete gathered weight
    consumed = [torch.cuda.Event() for _ in range(n_wbuf)]   # the GEMM that read buffer b has finished
    state = {"next": 0, "primed": False}
    gemm_events = []

    def prefetch_weight(w_dev):
        """Quantize this rank's weight rows and all-gather them into the next buffer (side stream)."""
        b = state["next"]
        comm_stream.wait_stream(torch.cuda.current_stream(dev))   # w_dev is ready
        comm_stream.wait_event(consumed[b])
        with torch.cuda.stream(comm_stream):
            if sym is not None:
                # One fence per step, after the scatter: the readers of buffer b start once every rank's
                # rows have landed. No fence is needed before overwriting b on the peers, because there
                # are three buffers: b was last read by the GEMM two steps back, and this stream has
                # already passed the fence of the previous prefetch, which no rank reaches before its
                # own copy of that GEMM has finished (each rank's prefetch waits for its main stream).
                sym.quantize_scatter(w_dev, b)
                sym.fence()
            else:
                wq, ws = gn_kernels.quantize_rowwise(w_dev)
                dist.all_gather_into_tensor(wq_full[b], wq)
                dist.all_gather_into_tensor(ws_full[b], ws)
                wq.record_stream(comm_stream)
                ws.record_stream(comm_stream)
            gathered[b].record(comm_stream)
        state["next"] = (b + 1) % n_wbuf
        return b

    def step(a_dev, w_dev, record_gemm=False):
        if world > 1:
            if not state["primed"]:
                state["ready"] = prefetch_weight(w_dev)
                state["primed"] = True
            b = state["ready"]
            state["ready"] = prefetch_weight(w_dev)     # next step's weight, overlapped with this step
            aq, as_ = gn_kernels.quantize_rowwise(a_dev)
            torch.cuda.current_stream(dev).wait_event(gathered[b])
            wq_all, ws_all = wq_full[b], ws_full[b]
        else:
            b = -1
            wq_all, ws_all = gn_kernels.quantize_rowwise(w_dev)
            aq, as_ = gn_kernels.quantize_rowwise(a_dev)
        if record_gemm:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        out = gn_kernels.scaled_mm(aq, wq_all.T, as_, ws_all.view(1, -1))
        if record_gemm:
            e1.record()
            gemm_events.append((e0, e1))
        if b >= 0:
            consumed[b].record()
        return out

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing ---------------------------------------------------------------
    # The clock sampler (nvidia-smi) is started first and given time to attach: its start-up stalls
    # the GPU for milliseconds. Warm-up then runs for at least 0.3 s so the clocks the timed region
    # sees are the ones the sampler records under load.
    sampler = ClockSampler(local_rank)
    if rank == 0 and not args.no_clock_sampler:
        sampler.start()
        time.sleep(0.2)
    sync_all()
    # The collector runs now and stays off until the timed region is over: a collection between warm-up
    # and the timed steps would leave the GPU idle for tens of milliseconds, the power controller would
    # hand the clocks back, and the region would measure that transient instead of the loaded state.
    gc.collect()
    gc.disable()
    warm_steps = 0
    t_warm = time.perf_counter()
    chunk = max(args.warmup, 3)
    while True:
        for _ in range(chunk):
            step(A, W)
        warm_steps += chunk
        torch.cuda.synchronize()
        if warm_steps == chunk:
            sampler.mark()          # from here on the GPU is under this workload's load
        more = 1 if (time.perf_counter() - t_warm) < args.min_warmup_seconds else 0
        if world > 1:  # every rank must run the same number of steps (the step holds a collective)
            flag = torch.tensor([more], dtype=torch.int32, device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            more = int(flag.item())
        if not more:
            break
    sync_all()
    # The barrier + synchronize above leave the GPU idle for milliseconds; two more untimed steps put it
    # back under load so the first timed step does not pay the ramp-up.
    #
    # A timed region is exactly --steps steps between two events. On these shared hosts a region is now
    # and then hit by a stall of tens of milliseconds that has nothing to do with the work (one GEMM of
    # 0.3 ms measured at 53 ms with every other launch normal). Such a region is measured again, at most
    # twice: it is rejected when its slowest GEMM took more than 5x the median GEMM of the region, on any
    # rank. The line reports how many regions were timed and what the rejected ones measured.
    discarded = []
    for attempt in range(3):
        # Clock samples bracket the region under the same continuous load instead of falling inside it:
        # an NVML query stalls the GPU's queued work for milliseconds to tens of milliseconds (with a
        # query placed inside every region, 5 of 6 regions had such a hole; with none, 0 of 3). One sample
        # is taken while untimed lead-in steps run, the others while untimed tail steps run right after
        # the region's last kernel has finished.
        sampler.pause()
        for _ in range(4):
            step(A, W)
        sampler.sample_now(1)
        # ... and that query (or the hole that got the previous region rejected) may have left the GPU
        # idle long enough for the power controller to hand the clocks back: 400 more untimed steps
        # (a fixed count, the same on every rank; about 0.2 s) bring back the loaded state the timed
        # steps are meant to see.
        for _ in range(400):
            step(A, W)
        warm_steps += 404
        gemm_events.clear()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.steps):
            out = step(A, W, record_gemm=True)
        stop.record()
        for _ in range(12):
            step(A, W)             # keeps the GPU under the same load while the clocks are read
        while not stop.query():
            time.sleep(0)
        sampler.sample_now(2)
        sampler.resume()
        sync_all()
        ms_total = max_over_ranks(start.elapsed_time(stop))
        gemm_times = [e0.elapsed_time(e1) for e0, e1 in gemm_events]
        gemm_ms_median = statistics.median(gemm_times)
        disturbed = max_over_ranks(1.0 if max(gemm_times) > 5.0 * gemm_ms_median else 0.0) > 0.0
        if not disturbed or attempt == 2:
            break
        discarded.append({"ms_per_step": ms_total / args.steps, "slowest_gemm_ms": max(gemm_times), "median_gemm_ms": gemm_ms_median})
    gc.enable()
    ms_per_step = ms_total / args.steps
    gemm_ms = statistics.mean(gemm_times)
    status = _native.device_status()
    if status != 0:
        raise SystemExit(f"a kernel reported a bounded wait that ran out (status {status:#x})")
    if world > 1:
        # the pipelined result of the last step against the same product through quantize + NCCL all-gather
        from gn_kernels.sharded import all_gather_quantized_rows
        wq_ref, ws_ref = all_gather_quantized_rows(*gn_kernels.quantize_rowwise(W), total_rows=gN)
        aq_ref, as_ref = gn_kernels.quantize_rowwise(A)
        ref = gn_kernels.scaled_mm(aq_ref, wq_ref.T, as_ref, ws_ref.view(1, -1))
        same = torch.tensor([1 if torch.equal(out, ref) else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        if int(same.item()) != 1:
            raise SystemExit("the pipelined multi-GPU step disagrees with quantize + all-gather + GEMM run in order")
        del wq_ref, ws_ref, aq_ref, as_ref, ref

    # ---- end to end through the public API from pinned host buffers -----------------------------
    # Every step copies its two bf16 inputs from pinned host memory and its bf16 result back. The
    # copies run on their own streams with double-buffered device tensors, so the upload of step i+1
    # and the download of step i-1 overlap the kernels of step i (PCIe is full duplex); all of it is
    # inside the timed region.
    h2d_stream, d2h_stream = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    main_stream = torch.cuda.current_stream(dev)
    a_bufs = [torch.empty_like(A) for _ in range(2)]
    w_bufs = [torch.empty_like(W) for _ in range(2)]
    o_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    uploaded = [torch.cuda.Event() for _ in range(2)]
    inputs_free = [torch.cuda.Event() for _ in range(2)]
    downloaded = [torch.cuda.Event() for _ in range(2)]
    keep = [None, None]
    e2e_count = {"i": 0}

    def e2e_step():
        i = e2e_count["i"]
        b = i & 1
        with torch.cuda.stream(h2d_stream):
            h2d_stream.wait_event(inputs_free[b])          # the step that last read these buffers is done
            a_bufs[b].copy_(A_host, non_blocking=True)
            w_bufs[b].copy_(W_host, non_blocking=True)
            uploaded[b].record(h2d_stream)
        main_stream.wait_event(uploaded[b])
        o = step(a_bufs[b], w_bufs[b])
        inputs_free[b].record(main_stream)
        ready = torch.cuda.Event()
        ready.record(main_stream)
        with torch.cuda.stream(d2h_stream):
            d2h_stream.wait_event(ready)
            d2h_stream.wait_event(downloaded[b])           # the host buffer's previous download is done
            o_hosts[b].copy_(o, non_blocking=True)
            downloaded[b].record(d2h_stream)
        o.record_stream(d2h_stream)
        keep[b] = o
        e2e_count["i"] = i + 1

    def e2e_drain():
        main_stream.wait_stream(h2d_stream)
        main_stream.wait_stream(d2h_stream)

    for _ in range(3):
        e2e_step()
    e2e_drain()
    sync_all()
    e2e_steps = max(3, min(args.steps, 10))
    e2e_regions = []
    for _ in range(3):   # three regions, the median is reported; all are in the line
        sampler.pause()
        s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for _ in range(e2e_steps):
            e2e_step()
        e2e_drain()                                        # the last result has reached the host
        t2.record()
        sampler.resume()
        sync_all()
        e2e_regions.append(max_over_ranks(s2.elapsed_time(t2)) / e2e_steps)
    e2e_ms = statistics.median(e2e_regions)
    clocks = sampler.stop() if rank == 0 else None

    # The metric's second half on the same ranks: INT8 mixed-precision training throughput of the 1.1B decoder
    # (FSDP2 with the INT8 weight all-gather when there are several ranks). A failure here must not lose the line.
    train_obj = None
    if not args.no_train_line and (gM, gN, gK) == (8192, 8192, 8192):
        try:
            del a_bufs, w_bufs, keep, wq_full, ws_full
            sym = None
            gc.collect()
            torch.cuda.empty_cache()
            _native.check(_native.load().qt_set_gemm_sm_margin(0))
            t = train_measure("train-1b", "mixed_precision", "fsdp", 3, 3, rank, local_rank, world)
            train_obj = {k: t[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "warmup", "loss", "max_memory_gb", "config")}
        except Exception as exc:   # noqa: BLE001
            train_obj = {"error": f"{type(exc).__name__}: {str(exc)[:300]}"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    flops = 2.0 * gM * gN * gK
    value = world * flops / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
    hbm_peak, bf16_peak, peak_kind = measured_peaks()
    # kind::i8 issues at twice the bf16 rate and the driver measures bf16 only. The GEMM is timed inside a
    # long step in the loaded, power-capped state, so the denominator is the SUSTAINED bf16 figure x 2; the
    # fraction of the burst figure x 2 is given beside it.
    bf16_sustained, sustained_kind = measured_sustained_bf16()
    int8_peak = 2.0 * bf16_sustained
    int8_peak_burst = 2.0 * bf16_peak
    achieved = flops / (gemm_ms * 1e-3) / 1e12
    # dram__bytes_read.sum + dram__bytes_write.sum of one 8192^3 launch of this kernel under ncu (a separate
    # run: counters cannot be read inside a timed run); None for shapes that were not captured
    traffic = 461.3e6 if (gM, gN, gK) == (8192, 8192, 8192) else None

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1 and gM == gN == gK:
        tops, threads, dt = time_cpu_path(S, 3 if S >= 8192 else 5, 1)
        cpu_baseline = {"value": tops, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": f"3 full passes of the {S}^3 workload after 1 warm-up ({dt:.2f} s each), torch eager quantize + torch._int_mm on the host"}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "lead_in_steps": warm_steps - max(args.warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8", "data": "synthetic",
        "config": {
            "workload": workload_name(gM, gN, gK),
            "weight_all_gather": ("none (1 GPU)" if world == 1 else
                                  "fused into the quantize kernel: int8 rows + bf16 scales stored into every rank's buffer over NVLink (peer-to-peer stores, symmetric memory), one step ahead on a side stream" if fused_gather else
                                  "int8 rows + bf16 scales over NCCL, prefetched one step ahead on a side stream"),
            "sm_margin": args.sm_margin,
            **({"gather_note": gather_note} if gather_note else {}),
            **({"host_buffers": numa_note} if numa_note else {}),
            "l2": f"inputs larger than L2 ({(gM + gN) * gK * 2 / 1e6:.0f} MB bf16 in, {(gM + gN) * gK / 1e6:.0f} MB int8 operands, {gM * gN * 2 / 1e6:.0f} MB out per step)",
            "value_is": "2*M*N*K * n_gpus / step time; the step includes both quantize kernels",
        },
        "gemm_only": {"tops": achieved, "ms": gemm_ms, "ms_median": gemm_ms_median, "ms_max": max(e0.elapsed_time(e1) for e0, e1 in gemm_events)},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                     "frac": achieved / int8_peak, "traffic": traffic,
                     "traffic_is": "DRAM bytes per launch from an ncu capture of this kernel at this shape (not measured in this run); algorithmic bytes 268.4e6",
                     "frac_of_nominal_4500_tops": achieved / NOMINAL_INT8_DENSE_TOPS,
                     "peak_is": f"2 x {sustained_kind} dense bf16 SUSTAINED ({bf16_sustained} TF/s: the GEMM is timed inside a long loaded step); "
                                f"nominal dense INT8 is {NOMINAL_INT8_DENSE_TOPS} TOPS",
                     "frac_of_burst": achieved / int8_peak_burst,
                     "burst_peak": int8_peak_burst,
                     "kernel": "gemm_kernel<int8, row/col-scaled, K-major A, K-major B>"},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": A_host.numel() * 2 + W_host.numel() * 2,
                "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": e2e_ms, "regions_ms_per_step": e2e_regions},
        "gpu_launches": 3 * args.steps,
        "timed_regions": {"measured": len(discarded) + 1, "rejected": discarded,
                          "rule": "a region whose slowest GEMM exceeds 5x its median GEMM is timed again (at most twice)"},
        "clocks": clocks,
    }
    if cpu_baseline is not None:
        line["cpu_baseline"] = cpu_baseline
    if train_obj is not None:
        line["train"] = train_obj
    if world == 1 and not args.no_quantize_lines:
        # the HBM-bound kernels of the path, each against the measured copy bandwidth (same entries as --workload quantize)
        del A, W, out
        torch.cuda.empty_cache()
        line["quantize"] = quantize_lines(32768, 2048, 20, dev)
    if world == 1 and not args.no_gemm_variants and (gM, gN, gK) == (8192, 8192, 8192):
        # the path's other GEMM forms at the same size (FP8, tile-scaled, the other layouts, raw INT8)
        torch.cuda.empty_cache()
        line["gemm_variants"] = gemm_variant_lines(dev)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
