"""Benchmark of the attention hot path: attention TFLOP/s (FLOPs = 4 * B * H * N^2 * d) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One STEP is one pass of the hot path over one batch: the attention calls of all layers of one forward of the
workload model, each layer reading its own packed qkv tensor (so consecutive launches never find their inputs in
L2). At N GPUs every rank runs the same step on its own images (image-wise sharding, no collective on the data
path) and the reported value is the whole-job aggregate, timed on the device as the maximum over ranks.

The JSON line carries, besides the contract's keys:
  roofline      tensor-pipe roofline of the attention kernel: achieved TFLOP/s per launch over the measured cuBLAS
                bf16 peak (MEASURED_PEAKS.json, else the fallback 1590 TFLOP/s)
  cpu_baseline  the reference's portable arithmetic (fp32 scaled_dot_product_attention on the host cores), timed on
                a bounded sample on rank 0
  e2e           the same metric through the public operator with HOST buffers: pinned-memory qkv copied to the
                device, attention, output copied back, every step
  regimes       the other benchmark shapes, device-timed: long-sequence TFLOP/s and short-sequence HBM GB/s
  model         ViT-L/14 518 px encoder around the kernel: images/s device-timed and end to end from host images
  partition     ViT-g/14 518 px, 256 images split image-wise over the ranks (strong scaling), gathered to rank 0 after
                the timed region

`--impl reference` times the reference's own CPU implementation of the path (see `oracle/portable_attention.py`)
on the same configuration and metric.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HEAD_DIM = 64
# Workload of the headline number: DINOv2 ViT-S/14 at 518x518 (N = 1 + 37 * 37), batch 8, fp16, 12 layers.
WORKLOAD = {"name": "dinov2-vits14-518px attention", "batch": 8, "heads": 6, "tokens": 1370, "layers": 12, "dtype": "fp16"}
# Device-timed side measurements (one layer each): the other shapes of the benchmark list.
REGIMES = (
    ("depth-anything-v2-l [4,16,1370,64] bf16", 4, 16, 1370, "bf16", None),
    ("sam-vit-b global [1,12,4096,64] fp16 + rel bias", 1, 12, 4096, "fp16", (64, 64)),
    ("dinov2-vitg14 [32,24,1370,64] bf16", 32, 24, 1370, "bf16", None),
    ("sam-vit-b windows [25,12,196,64] fp16 + rel bias", 25, 12, 196, "fp16", (14, 14)),
    ("vit-b16 [256,12,197,64] fp16", 256, 12, 197, "fp16", None),
    ("vit-b16 [1,12,197,64] fp16", 1, 12, 197, "fp16", None),
)
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0}
# Small single-kernel cases for profiler captures: `python bench.py --case NAME --launches L` launches the attention
# kernel L times on one set of buffers and exits (name -> batch, heads, tokens, dtype, rel grid).
CASES = {
    "dinov2-vits14": (8, 6, 1370, "fp16", None),
    "dav2-l": (4, 16, 1370, "bf16", None),
    "sam-global": (1, 12, 4096, "fp16", (64, 64)),
    "sam-windows": (25, 12, 196, "fp16", (14, 14)),
    "vit-b16-b256": (256, 12, 197, "fp16", None),
    "vit-b16-b1": (1, 12, 197, "fp16", None),
}
# The other kernels of the library, for the same purpose (name -> what is launched).
AUX_CASES = {
    "gemm-vitl-proj": "gemm [5480,1024] x [1024,1024]^T bf16 + bias, LayerScale, in-place residual (ViT-L/14 518 px, batch 4)",
    "gemm-vitl-fc1": "gemm [5480,1024] x [4096,1024]^T bf16 + bias, gelu (tanh form)",
    "gemm-vitl-qkv": "gemm [5480,1024] x [3072,1024]^T bf16 + bias",
    "gemm-4k": "gemm [4096,4096] x [4096,4096]^T bf16, no epilogue terms",
    "sam-rel-global": "sam_rel_terms of q [1,4096,12,64] fp16, 64 x 64 grid",
    "sam-rel-windows": "sam_rel_terms of q [25,196,12,64] fp16, 14 x 14 grid",
    "bias-swin": "attention [8,192,49,64] fp16 (Swin windows folded into the heads) + dense bias [1,192,49,56][..., :49] in tiles",
    "bias-1370": "attention [8,16,1370,64] fp16 + dense bias [1,16,1370,1376][..., :1370] in tiles",
    "rope-dinov3-vitl": "rope_qk_ of qkv [32,1029,3,16,64] fp16 in place (DINOv3 ViT-L/16 at 512 px): 270 MB read + written, time per launch reported",
}
# DRAM bytes of one launch of the headline kernel ([8,6,1370,64] fp16): dram__bytes_read.sum + dram__bytes_write.sum
# of one profiler capture of `python bench.py --case dinov2-vits14` (q, k, v are read once, 25.3 MB; the 8.4 MB output
# is still in L2 when the kernel ends). A profiler figure, not something this run measures: the line says so.
TRAFFIC_BYTES_PER_LAUNCH = 25.3e6
MIN_TIMED_SECONDS = 0.5  # the K-step region is repeated until this much device time has been measured


def attention_flops(b: int, h: int, n: int, nk: int | None = None) -> float:
    return 4.0 * b * h * n * (nk or n) * HEAD_DIM


def attention_bytes(b: int, h: int, n: int, rel: tuple[int, int] | None = None) -> float:
    """Algorithmic bytes of one call: q, k, v read once, o written once (2-byte elements), plus the bias terms."""
    extra = 2.0 * b * h * n * (rel[0] + rel[1]) if rel else 0.0
    return 8.0 * b * h * n * HEAD_DIM + extra


def load_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            data = json.loads(path.read_text())
            return {"bf16_tflops": float(data["bf16_tflops"]), "hbm_gbs": float(data["hbm_gbs"])}, "measured"
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    BAD = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20}
    NOTED = {"sw_power_cap": 0x4}

    def __init__(self, index: int) -> None:
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._dev, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001 - NVML is optional; absence is reported as null clocks
            self._nv = None

    def _sample(self) -> None:
        nv = self._nv
        self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._dev, nv.NVML_CLOCK_SM)))
        mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._dev))
        for name, bit in {**self.BAD, **self.NOTED}.items():
            if mask & bit:
                self.reasons.add(name)

    def _run(self) -> None:
        while not self._stop.is_set():
            try:
                self._sample()
            except Exception:  # noqa: BLE001
                return
            self._stop.wait(0.002)

    def __enter__(self) -> ClockSampler:
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc: object) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


class CpuReference:
    """The reference's portable arithmetic on the host: fp32 SDPA of `layers` layers of the workload shape, on
    buffers allocated (and touched) once."""

    def __init__(self, layers: int, threads: int) -> None:
        import torch

        from oracle.portable_attention import portable_attention

        torch.set_num_threads(threads)
        self.run = portable_attention
        self.layers, self.threads = layers, threads
        b, h, n = WORKLOAD["batch"], WORKLOAD["heads"], WORKLOAD["tokens"]
        gen = torch.Generator().manual_seed(0)
        self.qkv = [torch.randn(3, b, h, n, HEAD_DIM, generator=gen) for _ in range(layers)]
        self.flops = attention_flops(b, h, n) * layers
        self.sample = f"{layers} of {WORKLOAD['layers']} layers of [{b},{h},{n},{HEAD_DIM}] fp32 per pass"

    def one_pass(self) -> float:
        """Seconds of one pass over the sample."""
        t0 = time.perf_counter()
        for x in self.qkv:
            self.run(x[0], x[1], x[2])
        return time.perf_counter() - t0


def cpu_reference_tflops(layers: int, threads: int, *, warm: int = 2, runs: int = 5) -> tuple[float, float, str]:
    """(TFLOP/s, seconds per pass, description of the sample): median of `runs` passes after `warm` warm-ups."""
    ref = CpuReference(layers, threads)
    for _ in range(warm):
        ref.one_pass()
    sec = statistics.median(ref.one_pass() for _ in range(runs))
    return ref.flops / sec / 1e12, sec, f"{ref.sample}, median of {runs} passes after {warm} warm-ups"


def base_line(args: argparse.Namespace) -> dict:
    b, h, n = WORKLOAD["batch"], WORKLOAD["heads"], WORKLOAD["tokens"]
    return {
        "metric": "attention_tflops",
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "fp16",
        "data": "synthetic",
        "config": {
            "workload": f"{WORKLOAD['name']}: {WORKLOAD['layers']} layers of q,k,v [{b},{h},{n},{HEAD_DIM}] fp16 per GPU, "
            "strided views of packed qkv",
            "flops_per_step_per_gpu": attention_flops(b, h, n) * WORKLOAD["layers"],
            "l2": "each layer has its own 50 MB qkv and 17 MB output; a step touches 0.8 GB, larger than the 126 MB L2",
            "parallelism": f"image-wise shards, {args.gpus} replica(s), no data-path collective",
        },
    }


def run_reference(args: argparse.Namespace) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    layers = 2  # bounded sample of the 12-layer step; throughput is per FLOP, so the sample needs no scaling
    ref = CpuReference(layers, threads)  # buffers are allocated and first touched here, outside every timed pass
    for _ in range(max(1, args.warmup)):
        ref.one_pass()
    t0 = time.perf_counter()
    passes = [ref.one_pass() for _ in range(max(1, args.steps))]
    elapsed = time.perf_counter() - t0
    tflops = ref.flops / statistics.median(passes) / 1e12
    line = base_line(args)
    line.update(
        impl="reference",
        value=tflops,
        ms_per_step=elapsed / max(1, args.steps) * 1e3,
        dtype="f32",
        cpu_baseline={
            "value": tflops,
            "unit": "TFLOP/s",
            "cores": threads,
            "kind": "port",
            "sample": f"{layers} of {WORKLOAD['layers']} layers per step, same buffers every step, median step: fp32 torch "
            "scaled_dot_product_attention on the host, the call the reference's portable backend makes",
        },
        e2e={"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        gpu_launches=0,
    )
    print(json.dumps(line))


def model_throughput(torch, ff, world: int, timed) -> dict | None:  # noqa: ANN001
    """images/s of the kernels-mode ViT-L/14 encoder at 518 px, batch 4 per GPU (aggregate over ranks, weak scaling),
    device-timed with the images resident, and end to end: images from pinned host memory in, features to pinned
    host memory out, every forward."""
    from fastforks_b200.vit import CONFIGS, ViTEncoder, seeded_state

    cfg = CONFIGS["dinov2-vitl14"]
    batch, side, steps = 4, 518, 5
    enc = ViTEncoder(cfg, seeded_state(cfg, 0), device="cuda", dtype=torch.bfloat16)
    host_images = torch.rand(batch, 3, side, side, generator=torch.Generator().manual_seed(1)).pin_memory()
    images = host_images.cuda()
    host_out = torch.empty(batch, cfg.tokens(side, side), cfg.dim, dtype=torch.bfloat16).pin_memory()
    out = None
    for _ in range(3):
        out = enc(images)

    def forward() -> None:
        enc(images)

    def forward_e2e() -> None:
        host_out.copy_(enc(host_images.cuda(non_blocking=True)), non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the features are in host memory when the call returns

    ms = timed(forward, steps)
    forward_e2e()
    ms_e2e = timed(forward_e2e, steps)
    own = ViTEncoder(cfg, seeded_state(cfg, 0), device="cuda", dtype=torch.bfloat16, fuse_plain=True)
    for _ in range(2):
        own(images)
    ms_own = timed(lambda: own(images), steps)
    del own
    # The launch-bound configuration (one image of ViT-B/16 at 224 px, 197 tokens): the forward as a stream of launches
    # and replayed from a CUDA graph.
    small_cfg = CONFIGS["vit-b16"]
    small = ViTEncoder(small_cfg, seeded_state(small_cfg, 0), device="cuda", dtype=torch.float16)
    one = torch.rand(1, 3, 224, 224, generator=torch.Generator().manual_seed(2)).half().cuda()
    cache = ff.GraphCache(small)
    for _ in range(3):
        cache(one)
    small_steps = 20
    ms_small_eager = timed(lambda: small(one), small_steps)
    ms_small_graph = timed(lambda: cache(one), small_steps)
    if ff.device_status() != 0 or not bool(torch.isfinite(out).all()):
        return None
    return {
        "launch_bound": {
            "name": "vit-b16 at 224 px, fp16, one image (197 tokens)",
            "ms_per_forward_eager": ms_small_eager / small_steps,
            "ms_per_forward_cuda_graph": ms_small_graph / small_steps,
        },
        "name": "dinov2-vitl14 (Depth-Anything-V2-L encoder) at 518 px, bf16",
        "batch_per_gpu": batch,
        "images_per_s": batch * steps * world / (ms * 1e-3),
        "ms_per_forward": ms / steps,
        "attention_gflop_per_image": enc.attention_flops(1, side, side) / 1e9,
        "linear_layers": "proj, fc1, fc2 on this library's GEMM with fused epilogue; qkv (bias only) on torch's library GEMM",
        "images_per_s_every_linear_layer_own_gemm": batch * steps * world / (ms_own * 1e-3),
        "e2e": {
            "images_per_s": batch * steps * world / (ms_e2e * 1e-3),
            "h2d_bytes_per_forward": host_images.numel() * 4,
            "d2h_bytes_per_forward": host_out.numel() * 2,
        },
    }


PARTITION = {"model": "dinov2-vitg14", "images": 256, "side": 518, "chunk": 16, "check": 3}


def partition_throughput(torch, ff, dist, world: int, rank: int, timed) -> dict | None:  # noqa: ANN001
    """The partition the reference's multi-GPU rule gives (one process per GPU, images split between them, no
    communication while a model runs: docs/usage.md:658-662, src/fastforks/_core/model.py:1006-1015): DINOv2 ViT-g/14
    (`vit_giant2`, SwiGLU) at 518 px, bf16, 256 seeded images as contiguous ranges of 256 / G images per rank, run in
    chunks of 16. Strong scaling: the job is the same at every G. The outputs are gathered to rank 0 AFTER the timed
    region, where a few images are checked against the same images run alone."""
    from fastforks_b200 import sharding
    from fastforks_b200.vit import CONFIGS, ViTEncoder, seeded_state

    cfg = CONFIGS[PARTITION["model"]]
    total, side, chunk = PARTITION["images"], PARTITION["side"], PARTITION["chunk"]
    enc = ViTEncoder(cfg, seeded_state(cfg, 0), device="cuda", dtype=torch.bfloat16)
    mine = sharding.image_range(total, world, rank)

    def image(i: int):  # noqa: ANN202 - every rank can make any image: seeded by its index
        return torch.rand(3, side, side, generator=torch.Generator().manual_seed(10_000 + i))

    images = torch.stack([image(i) for i in mine]).cuda().to(torch.bfloat16)
    pooled = torch.empty(len(mine), 2 * cfg.dim, device="cuda", dtype=torch.float32)

    def job() -> None:
        for at in range(0, len(mine), chunk):
            tokens = enc(images[at : at + chunk])
            # what `features` models hand back: class token and mean patch token (src/fastforks/features/models/dinov2)
            pooled[at : at + chunk] = torch.cat([tokens[:, 0], tokens[:, 1:].mean(1)], -1).float()

    job()  # warm-up: cuBLAS plans, position table
    ms = timed(job, 1)
    if ff.device_status() != 0:
        return None
    t0 = time.perf_counter()
    gathered = sharding.gather_to_rank0(pooled, total) if dist is not None else pooled
    torch.cuda.synchronize()
    gather_ms = (time.perf_counter() - t0) * 1e3
    result = {
        "name": f"{PARTITION['model']} at {side} px, bf16: {total} images split image-wise over {world} GPU(s), chunks of {chunk}",
        "scaling": "strong",
        "images": total,
        "images_per_s": total / (ms * 1e-3),
        "ms_job": ms,
        "gather_to_rank0_ms_outside_timing": gather_ms,
    }
    if rank == 0:
        picks = [0, total // 2, total - 1][: PARTITION["check"]]
        cos = []
        for i in picks:
            alone = enc(image(i)[None].cuda().to(torch.bfloat16))
            ref = torch.cat([alone[:, 0], alone[:, 1:].mean(1)], -1).float()[0]
            cos.append(float(torch.nn.functional.cosine_similarity(ref, gathered[i], dim=0)))
        result["cosine_vs_same_image_alone_min"] = min(cos)
        result["finite"] = bool(torch.isfinite(gathered).all())
    del enc, images
    torch.cuda.empty_cache()
    return result


def time_launches(fn, reps: int, torch) -> float:  # noqa: ANN001
    """Average milliseconds of `fn()` over `reps` back-to-back calls, CUDA events on the current stream."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def run_ours(args: argparse.Namespace) -> None:  # noqa: PLR0915
    import torch

    import fastforks_b200 as ff

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            msg = f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks (WORLD_SIZE is 1)"
            raise SystemExit(msg)
        args.gpus = world
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist

        from datetime import timedelta

        # A finite limit on every collective and barrier: a rank that is gone ends the others with an error.
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=timedelta(seconds=180))
    ff.resolve_mode("kernels")  # raises when the CUDA library or a B200 is missing: no fallback is timed

    b, h, n, layers = WORKLOAD["batch"], WORKLOAD["heads"], WORKLOAD["tokens"], WORKLOAD["layers"]
    gen = torch.Generator().manual_seed(1234 + rank)
    host_qkv = [torch.randn(b, n, 3, h, HEAD_DIM, generator=gen).half().pin_memory() for _ in range(layers)]
    dev_qkv = [x.cuda(non_blocking=True) for x in host_qkv]
    dev_out = [torch.empty(b, n, h, HEAD_DIM, dtype=torch.float16, device="cuda") for _ in range(layers)]
    host_out = [torch.empty(b, n, h, HEAD_DIM, dtype=torch.float16).pin_memory() for _ in range(layers)]
    views = [x.unbind(2) for x in dev_qkv]
    scale = HEAD_DIM**-0.5
    torch.cuda.synchronize()

    def step() -> None:
        for (q, k, v), o in zip(views, dev_out):
            ff.attention(q, k, v, scale=scale, layout="bnhd", out=o)

    host_attn = ff.HostAttention()

    def step_e2e() -> None:
        # Host buffers in, host buffers out, through the package's host-operand operator: every layer's packed qkv is
        # uploaded from pinned memory, its attention computed and its output downloaded; uploads, kernels and
        # downloads of neighbouring layers overlap on three streams. Returns when every output is in host memory.
        host_attn(host_qkv, host_out, scale)

    def barrier() -> None:
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int) -> float:  # noqa: ANN001
        """Milliseconds for `steps` calls of fn, device-timed, max over ranks."""
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(3, args.warmup)):
        step()
    # The K-step region is timed again and again until at least MIN_TIMED_SECONDS of device time are measured (every
    # rank sees the same all-reduced times, so all ranks stop together); the clocks are sampled over exactly these
    # regions. Reported: the median region, with the spread of all of them.
    regions: list[float] = []
    with ClockSampler(local) as clocks:
        while len(regions) < 3 or (sum(regions) < MIN_TIMED_SECONDS * 1e3 and len(regions) < 1000):
            regions.append(timed(step, args.steps))
    total_ms = statistics.median(regions)
    status = ff.device_status()
    if status != 0:
        msg = f"a kernel gave up a bounded wait (status {status}); the timing is void"
        raise SystemExit(msg)

    for _ in range(2):
        step_e2e()
    e2e_steps = max(1, min(args.steps, 10))
    e2e_ms = timed(step_e2e, e2e_steps)

    flops_step = attention_flops(b, h, n) * layers
    value = flops_step * args.steps * world / (total_ms * 1e-3) / 1e12
    e2e_value = flops_step * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
    per_launch_ms = total_ms / (args.steps * layers)
    achieved = attention_flops(b, h, n) / (per_launch_ms * 1e-3) / 1e12
    peaks, peak_kind = load_peaks()

    line = base_line(args)
    line.update(
        value=value,
        ms_per_step=total_ms / args.steps,
        images_per_s=b * world * args.steps / (total_ms * 1e-3),
        roofline={
            "bound": "tensor",
            "achieved": achieved,
            "peak": peaks["bf16_tflops"],
            "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16_tflops"],
            "traffic": TRAFFIC_BYTES_PER_LAUNCH,
            "traffic_source": "profile (one profiler capture of this kernel on this shape, not measured by this run)",
            "algorithmic_bytes": attention_bytes(b, h, n),
            "peak_source": f"{peak_kind} (cuBLAS bf16 burst)",
            "kernel": "attn_fwd_kernel<half, no bias>",
            "us_per_launch": per_launch_ms * 1e3,
        },
        e2e={
            "value": e2e_value,
            "unit": "TFLOP/s",
            "h2d_bytes_per_step": sum(x.numel() * 2 for x in host_qkv),
            "d2h_bytes_per_step": sum(x.numel() * 2 for x in host_out),
        },
        gpu_launches=args.steps * layers,
        clocks=clocks.summary(),
        timed_regions={
            "count": len(regions),
            "seconds": sum(regions) * 1e-3,
            "ms_min": min(regions),
            "ms_median": total_ms,
            "ms_max": max(regions),
            "spread": (max(regions) - min(regions)) / total_ms,
        },
    )

    # Whole-model throughput of the caller of the hot path: the ViT-L/14 encoder of Depth-Anything-V2-L / DINOv2-L at
    # 518 px (N = 1370, 24 layers, 16 heads), bf16, random-init weights, on every rank's own images. GEMMs, LayerNorm
    # and GELU are torch library calls; the attention is this repository's kernel.
    model = model_throughput(torch, ff, world, timed)
    if model is not None:
        line["model"] = model
    torch.cuda.empty_cache()
    # The partition the benchmark list names: ViT-g/14, 256 images split image-wise over the ranks (strong scaling).
    if not args.skip_partition:
        partition = partition_throughput(torch, ff, dist, world, rank, timed)
        if partition is not None:
            line["partition"] = partition

    if rank == 0:
        regimes = {}
        for name, rb, rh, rn, rdt, rel in REGIMES:
            dt = torch.float16 if rdt == "fp16" else torch.bfloat16
            copies = max(2, int(300e6 // attention_bytes(rb, rh, rn, rel)) + 1)  # rotate buffers: inputs larger than L2
            copies = min(copies, 64)
            qkvs = [torch.randn(rb, rn, 3, rh, HEAD_DIM, device="cuda").to(dt) for _ in range(copies)]
            outs = [torch.empty(rb, rn, rh, HEAD_DIM, device="cuda", dtype=dt) for _ in range(copies)]
            rels = None
            if rel:
                rels = [
                    (torch.randn(rb, rh, rn, rel[0], device="cuda").to(dt), torch.randn(rb, rh, rn, rel[1], device="cuda").to(dt))
                    for _ in range(copies)
                ]
            state = {"i": 0}

            def call(qkvs=qkvs, outs=outs, rels=rels, state=state, copies=copies) -> None:  # noqa: ANN001
                i = state["i"] = (state["i"] + 1) % copies
                q, k, v = qkvs[i].unbind(2)
                ff.attention(q, k, v, scale=scale, layout="bnhd", out=outs[i], rel=None if rels is None else rels[i])

            ms = time_launches(call, 40, torch)
            regimes[name] = {
                "us_per_launch": ms * 1e3,
                "tflops": attention_flops(rb, rh, rn) / (ms * 1e-3) / 1e12,
                "frac_tensor_peak": attention_flops(rb, rh, rn) / (ms * 1e-3) / 1e12 / peaks["bf16_tflops"],
                "hbm_gbs": attention_bytes(rb, rh, rn, rel) / (ms * 1e-3) / 1e9,
                "frac_hbm_peak": attention_bytes(rb, rh, rn, rel) / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            }
            del qkvs, outs, rels
        line["regimes"] = regimes
        line["peaks"] = {**peaks, "source": peak_kind}
        if world == 1:
            threads = os.cpu_count() or 1
            tflops, sec, sample = cpu_reference_tflops(2, threads)
            line["cpu_baseline"] = {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_case(args: argparse.Namespace) -> None:
    """Launch one named case `--launches` times without timing: the command profiler captures run."""
    import torch

    import fastforks_b200 as ff

    if args.case in AUX_CASES:
        gen = torch.Generator(device="cuda").manual_seed(0)

        def rnd(*shape: int, dt: torch.dtype = torch.bfloat16, mag: float = 1.0) -> torch.Tensor:
            return (torch.randn(*shape, device="cuda", generator=gen) * mag).to(dt)

        if args.case.startswith("gemm"):
            m, n, k = {"gemm-vitl-proj": (5480, 1024, 1024), "gemm-vitl-fc1": (5480, 4096, 1024), "gemm-vitl-qkv": (5480, 3072, 1024),
                       "gemm-4k": (4096, 4096, 4096)}[args.case]  # fmt: skip
            x, w, bias, res = rnd(m, k), rnd(n, k, mag=k**-0.5), rnd(n), rnd(m, n)
            scale = torch.rand(n, device="cuda", generator=gen) + 0.5
            for _ in range(args.launches):
                if args.case == "gemm-vitl-proj":
                    ff.gemm(x, w, bias, scale=scale, res=res, out=res)
                elif args.case == "gemm-vitl-fc1":
                    ff.gemm(x, w, bias, act=ff.ACT_GELU_TANH)
                elif args.case == "gemm-vitl-qkv":
                    ff.gemm(x, w, bias)
                else:
                    ff.gemm(x, w)
        elif args.case.startswith("bias"):
            b, h, n = (8, 192, 49) if args.case == "bias-swin" else (8, 16, 1370)
            qkv = rnd(b, n, 3, h, HEAD_DIM, dt=torch.float16)
            q, k, v = (x.transpose(1, 2) for x in qkv.unbind(2))
            bias = rnd(1, h, n, (n + 7) // 8 * 8, dt=torch.float16)[..., :n]
            times = {}
            for name, mask in (("none", None), ("tiles", bias)):
                ff.scaled_dot_product_attention(q, k, v, attn_mask=mask)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.launches):
                    ff.scaled_dot_product_attention(q, k, v, attn_mask=mask)
                e1.record()
                torch.cuda.synchronize()
                times[name] = e0.elapsed_time(e1) / args.launches * 1e3
            print(json.dumps({"case": args.case, "what": AUX_CASES[args.case], "launches": args.launches, "us_per_launch_no_bias": times["none"],
                              "us_per_launch_bias_tiles": times["tiles"], "status": ff.device_status()}))  # fmt: skip
            return
        elif args.case.startswith("rope"):
            qkv = rnd(32, 5 + 32 * 32, 3, 16, HEAD_DIM, dt=torch.float16)
            cs = ff.rope_table(32, 32, 100.0, "cuda")
            ff.rope_qk_(qkv, cs, q_scale=0.125)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.launches):
                ff.rope_qk_(qkv, cs, q_scale=0.125)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) / args.launches * 1e3
            moved = 2 * 2 * qkv.shape[0] * qkv.shape[1] * 16 * HEAD_DIM * 2  # q and k, read and written
            print(json.dumps({"case": args.case, "what": AUX_CASES[args.case], "launches": args.launches, "us_per_launch": us,
                              "gbs": moved / us / 1e3, "status": ff.device_status()}))  # fmt: skip
            return
        else:
            b, side = (1, 64) if args.case == "sam-rel-global" else (25, 14)
            q = rnd(b, side * side, 3, 12, HEAD_DIM, dt=torch.float16)[:, :, 0]
            pos_h, pos_w = rnd(2 * side - 1, HEAD_DIM, dt=torch.float16, mag=0.1), rnd(2 * side - 1, HEAD_DIM, dt=torch.float16, mag=0.1)
            for _ in range(args.launches):
                ff.sam_rel_terms(q, pos_h, pos_w, side)
        torch.cuda.synchronize()
        print(json.dumps({"case": args.case, "what": AUX_CASES[args.case], "launches": args.launches, "status": ff.device_status()}))
        return
    b, h, n, dtype, rel = CASES[args.case]
    dt = torch.float16 if dtype == "fp16" else torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn(b, n, 3, h, HEAD_DIM, device="cuda", generator=gen).to(dt)
    q, k, v = qkv.unbind(2)
    out = torch.empty(b, n, h, HEAD_DIM, device="cuda", dtype=dt)
    rels = None
    if rel:
        rels = tuple(torch.randn(b, h, n, r, device="cuda", generator=gen).to(dt) for r in rel)
    for _ in range(args.launches):
        ff.attention(q, k, v, layout="bnhd", out=out, rel=rels)
    torch.cuda.synchronize()
    print(json.dumps({"case": args.case, "launches": args.launches, "status": ff.device_status()}))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--case", choices=(*CASES, *AUX_CASES), default=None, help="launch one kernel case for a profiler and exit")
    ap.add_argument("--launches", type=int, default=4)
    ap.add_argument("--skip-partition", action="store_true", help="leave out the ViT-g/14 256-image partition leg")
    args = ap.parse_args()
    args.steps = max(1, args.steps)
    if args.case is not None:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
