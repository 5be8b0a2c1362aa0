"""Headline benchmark: MoE dispatch + combine all-to-all, DeepSeek-V3 shape.

One step = one ``AllToAll.dispatch`` (fp8 e4m3 payload + fp32 scale per 128
columns, 256 experts, top-8, hidden 7168, 128 tokens per GPU) followed by one
``AllToAll.combine`` (bf16 expert outputs -> bf16 tokens), the pair the
reference's own benchmark times (tests/bench_all_to_all.py:144-210).  Routing,
tokens and weights are synthetic.

    python bench.py --gpus 1 --steps 200 --warmup 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 \
        --master-addr 127.0.0.1 --master-port 29501 bench.py --gpus 8
    ... bench.py --impl reference --gpus 8      # the unmodified reference, same harness

Both arms run the same code in this file: the same tensors, the same timing
loops, the same rank barrier (an NCCL all-reduce of one word on the launching
stream) and the same JSON keys; only the ``AllToAll`` object differs.  The
reference arm imports nothing that maps this repository's native library.

Timing: every step is bracketed by CUDA events on the launching stream, after a
write of a 256 MiB buffer that flushes the 126 MB L2 and (for N > 1) the rank
barrier so that all ranks start together; per step the maximum over ranks is
taken, then the mean over the K timed steps gives ``ms_per_step`` and the
aggregate tokens/s; p50 values are reported next to it.  Rank 0 prints one JSON
line.
"""

from __future__ import annotations

import argparse
import json
import logging
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
_LOG = logging.getLogger("pplx_kernels_b200.bench")

# Published EP8 NVLink numbers of the reference (its README.md:60-81), in microseconds.
PUBLISHED_US = {1: {"dispatch": 41.6, "combine": 41.7}, 128: {"dispatch": 83.6, "combine": 102.3}}
PUBLISHED_WORLD = 8
# Peer-copy bandwidth per direction used for the NVLink floor when the run cannot measure it
# itself (a single GPU, or the measurement failed): GB/s of a large device-to-peer copy on an
# NVSwitch-connected B200.
NVLINK_GBS_DEFAULT = 770.0

# The two model shapes of the reference's benchmark (tests/bench_all_to_all.py:244-262):
# (experts, top-k, hidden); fp8 e4m3 tokens with one fp32 scale per 128 columns, bf16 results.
SHAPES = {"r1": (256, 8, 7168), "v2lite": (64, 6, 2048)}

METRIC = ("MoE dispatch+combine tokens/s (DeepSeek-V3 shape: 256 experts, top-8, hidden 7168, "
          "fp8 dispatch + bf16 combine)")
DTYPE = "fp8_e4m3 dispatch (fp32 scale per 128) / bf16 combine"
DATA = "synthetic (uniform random distinct top-8 routing, random tokens, softmax weights)"


def _peaks() -> dict:
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f)
    except OSError:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "fallback": True}


# File descriptor of the real standard output.  main() points descriptor 1 at standard error
# for the duration of the run, so that whatever native libraries print (NCCL's version banner,
# for one) does not land between the caller and the one JSON line it parses.
_RESULT_FD = 1


def _emit(line: dict) -> None:
    sys.stdout.flush()
    os.write(_RESULT_FD, (json.dumps(line) + "\n").encode())


def _env_rank() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def _repo_native_mapped() -> bool:
    """True if this process has mapped this repository's native library."""
    try:
        with open("/proc/self/maps") as f:
            return "libpplx_kernels_b200" in f.read()
    except OSError:
        return False


class PackedInputs:
    """One pinned host buffer and one device buffer holding [x | x_scale | indices | weights]
    of a step, so that the end-to-end path uploads a step's inputs with a single copy.  Both
    arms use it."""

    def __init__(self, inp, dev: torch.device) -> None:
        parts = [inp.x.view(torch.uint8).reshape(-1), inp.x_scale.view(torch.uint8).reshape(-1),
                 inp.indices.to(torch.int32).view(torch.uint8).reshape(-1),
                 inp.weights.view(torch.uint8).reshape(-1)]
        offs, total = [], 0
        for t in parts:
            offs.append(total)
            total += (t.numel() + 255) // 256 * 256
        self.host = torch.zeros(total, dtype=torch.uint8).pin_memory()
        for o, t in zip(offs, parts):
            self.host[o:o + t.numel()].copy_(t)
        self.dev = self.host.to(dev)
        self._routing_from = offs[2]
        m, hidden = inp.x.shape

        def view(buf: torch.Tensor, i: int, t: torch.Tensor, dtype: torch.dtype, shape) -> torch.Tensor:
            return buf[offs[i]:offs[i] + t.numel()].view(dtype).view(shape)

        shapes = [(inp.x.dtype, (m, hidden)), (torch.float32, tuple(inp.x_scale.shape)),
                  (torch.uint32, tuple(inp.indices.shape)), (torch.float32, tuple(inp.weights.shape))]
        self.x, self.x_scale, self.indices, self.weights = (
            view(self.dev, i, parts[i], dt, sh) for i, (dt, sh) in enumerate(shapes))
        # The same four tensors as views of the pinned host buffer (for a dispatch that reads
        # its inputs from host memory itself).
        self.h_x, self.h_x_scale, self.h_indices, self.h_weights = (
            view(self.host, i, parts[i], dt, sh) for i, (dt, sh) in enumerate(shapes))

    def upload(self) -> None:
        self.dev.copy_(self.host, non_blocking=True)

    def upload_routing(self) -> None:
        """Copies only indices and weights (a few KiB, adjacent in the buffer)."""
        self.dev[self._routing_from:].copy_(self.host[self._routing_from:], non_blocking=True)

    def nbytes(self) -> int:
        return self.host.numel()


class Arm:
    """The tensors of one benchmark arm and its all-to-all object.

    `kind` is "ours", "ref-intranode" or "ref-internode"; everything except the construction
    of ``self.ata`` is the same for all three.
    """

    def __init__(self, kind: str, tokens: int, rank: int, world: int, dev: torch.device,
                 shape: str = "r1", zipf: float = 0.0) -> None:
        from pplx_kernels_b200.utils.testing import MoEConfig, make_rank_inputs

        self.kind, self.rank, self.world, self.device, self.tokens = kind, rank, world, dev, tokens
        experts, topk, hidden = SHAPES[shape]
        cfg = MoEConfig(num_experts=experts, experts_per_token=topk, hidden_dim=hidden,
                        max_num_tokens=tokens, in_dtype=torch.float8_e4m3fn,
                        out_dtype=torch.bfloat16)
        self.cfg = cfg
        nle = cfg.num_experts // world
        inp = make_rank_inputs(cfg, torch.Generator().manual_seed(1000 + rank), num_tokens=tokens,
                               softmax_weights=True, zipf=zipf)
        if rank == 0 and _LOG.isEnabledFor(logging.DEBUG):
            from pplx_kernels_b200.utils.logging_utils import describe_routing

            _LOG.debug("%s, %d tokens: rank 0 routes\n%s", kind, tokens,
                       describe_routing(inp.indices, cfg.num_experts, world))
        self.packed = PackedInputs(inp, dev)
        self.x, self.x_scale = self.packed.x, self.packed.x_scale
        self.indices, self.weights = self.packed.indices, self.packed.weights
        self.bound_m = torch.tensor([tokens], dtype=torch.int32, device=dev).view(torch.uint32)
        rows = tokens * world
        self.counts = torch.zeros(nle, dtype=torch.int32, device=dev)
        self.expert_x = torch.zeros(nle, rows, cfg.hidden_dim, dtype=torch.uint8,
                                    device=dev).view(cfg.in_dtype)
        self.expert_scale = torch.zeros(nle, rows, cfg.hidden_dim_scale, device=dev)
        self.expert_y = torch.randn(nle, rows, cfg.hidden_dim, device=dev).to(cfg.out_dtype)
        self.out = torch.zeros(tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=dev)
        self.h_out = torch.empty(tokens, cfg.hidden_dim, dtype=cfg.out_dtype).pin_memory()
        kwargs = dict(max_num_tokens=tokens, num_experts=cfg.num_experts,
                      experts_per_token=cfg.experts_per_token, rank=rank, world_size=world,
                      dp_size=1, hidden_dim=cfg.hidden_dim, hidden_dim_bytes=cfg.hidden_dim_bytes,
                      hidden_dim_scale_bytes=cfg.hidden_dim_scale_bytes)
        if kind == "ours":
            import pplx_kernels_b200 as pk

            self.ata = pk.AllToAll.intranode(**kwargs)
        else:
            from pplx_kernels.all_to_all import AllToAll as RefAllToAll  # the reference's class

            make = RefAllToAll.intranode if kind == "ref-intranode" else RefAllToAll.internode
            self.ata = make(**kwargs)

    def dispatch(self) -> None:
        self.ata.dispatch(self.counts, self.expert_x, self.expert_scale, self.x, self.x_scale,
                          self.indices, self.bound_m)

    def dispatch_from_host(self) -> None:
        """dispatch whose send reads tokens and scales from pinned host memory; the routing
        table (every block reads all of it) has been copied to the device."""
        p = self.packed
        self.ata.dispatch(self.counts, self.expert_x, self.expert_scale, p.h_x, p.h_x_scale,
                          self.indices, self.bound_m)

    def combine(self) -> None:
        self.ata.combine(self.out, self.indices, self.weights, self.expert_y, self.bound_m)

    def combine_to_host(self) -> None:
        """combine whose reduction writes the tokens straight into the pinned host buffer."""
        self.ata.combine(self.h_out, self.indices, self.weights, self.expert_y, self.bound_m)


    def upload(self) -> None:
        self.packed.upload()

    def download(self) -> None:
        self.h_out.copy_(self.out, non_blocking=True)

    def h2d_bytes(self) -> int:
        return self.packed.nbytes()

    def d2h_bytes(self) -> int:
        return self.h_out.numel() * self.h_out.element_size()

    def close(self) -> None:
        if self.kind == "ours":
            self.ata.check_status()
        self.ata.destroy()


class Harness:
    """Timing loops shared by both arms."""

    def __init__(self, world: int, dev: torch.device, steps: int, warmup: int) -> None:
        self.world, self.dev, self.steps, self.warmup = world, dev, steps, warmup
        self.flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
        self.sync_word = torch.zeros(1, device=dev)

    def rank_barrier(self) -> None:
        """Device-side barrier on the launching stream: an NCCL all-reduce of one word."""
        if self.world > 1:
            torch.distributed.all_reduce(self.sync_word)

    def max_over_ranks(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        return t

    def all_agree(self, ok: bool) -> bool:
        flag = torch.tensor([1.0 if ok else 0.0], device=self.dev)
        if self.world > 1:
            torch.distributed.all_reduce(flag, op=torch.distributed.ReduceOp.MIN)
        return flag.item() >= 1.0

    def time_pair(self, first, second, steps: int | None = None) -> torch.Tensor:
        """[steps, 3] microseconds (first, second, both) with an event between the two calls,
        max over ranks."""
        steps = steps or self.steps
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        for i in range(self.warmup + steps):
            self.flush.add_(1)
            self.rank_barrier()
            e = evs[i - self.warmup] if i >= self.warmup else None
            if e:
                e[0].record()
            first()
            if e:
                e[1].record()
            second()
            if e:
                e[2].record()
        torch.cuda.synchronize()
        t = torch.tensor([[e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2]),
                           e[0].elapsed_time(e[2])] for e in evs],
                         dtype=torch.float64, device=self.dev) * 1e3
        return self.max_over_ranks(t).cpu()

    def time_step(self, step, steps: int | None = None) -> torch.Tensor:
        """[steps] microseconds of `step()` with nothing recorded inside it, max over ranks."""
        steps = steps or self.steps
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(steps)]
        for i in range(self.warmup + steps):
            self.flush.add_(1)
            self.rank_barrier()
            e = evs[i - self.warmup] if i >= self.warmup else None
            if e:
                e[0].record()
            step()
            if e:
                e[1].record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) for a, b in evs], dtype=torch.float64,
                         device=self.dev) * 1e3
        return self.max_over_ranks(t).cpu()

    def time_graph(self, step) -> tuple[float | None, str]:
        """Mean microseconds of `step()` captured once and replayed as one CUDA graph."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph: torch.cuda.CUDAGraph | None = torch.cuda.CUDAGraph()
        why = ""
        try:
            with torch.cuda.graph(graph, stream=side):
                step()
        except Exception as exc:  # noqa: BLE001 - reported in the JSON line
            graph, why = None, f"capture failed: {type(exc).__name__}: {str(exc)[:120]}"
        torch.cuda.synchronize()
        if not self.all_agree(graph is not None):
            return None, why or "capture failed on another rank"
        return float(self.time_step(graph.replay).mean()), ""


def measure_arm(kind: str, h: Harness, tokens: int, rank: int, world: int, no_graph: bool) -> dict:
    """Every figure of one arm: kernel-only latencies at `tokens` and at 1 token per GPU, and
    the end-to-end step in every mode the arm supports."""
    arm = Arm(kind, tokens, rank, world, h.dev)

    def step() -> None:
        arm.dispatch()
        arm.combine()

    def step_e2e() -> None:
        arm.upload()
        arm.dispatch()
        arm.combine()
        arm.download()

    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    wall0 = time.perf_counter()
    t_pair = h.time_pair(arm.dispatch, arm.combine)
    t_step = h.time_step(step)
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    wall1 = time.perf_counter()
    modes: dict[str, float | None] = {
        "eager calls, copy engine both ways": float(h.time_step(step_e2e).mean())}
    graph_why = "disabled"
    if not no_graph:
        modes["one CUDA graph replay per step"], graph_why = h.time_graph(step_e2e)
    if kind == "ours":
        def step_host_out() -> None:
            arm.upload()
            arm.dispatch()
            arm.combine_to_host()

        def step_host_both() -> None:
            arm.packed.upload_routing()
            arm.dispatch_from_host()
            arm.combine_to_host()

        modes["eager calls, combine writes the tokens to pinned host memory"] = float(
            h.time_step(step_host_out).mean())
        try:
            modes["eager calls, dispatch reads the tokens from and combine writes the tokens to "
                  "pinned host memory (routing table copied)"] = float(h.time_step(step_host_both).mean())
            if not no_graph:
                modes["one CUDA graph replay per step, tokens read from and written to pinned "
                      "host memory (routing table copied)"], _ = h.time_graph(step_host_both)
        except RuntimeError as exn:  # an older native library without host-input support
            graph_why = (graph_why + "; " if graph_why else "") + f"host-input mode: {str(exn)[:100]}"
    res = {
        "latency_us": {str(tokens): {
            "dispatch_us_p50": float(t_pair[:, 0].median()),
            "combine_us_p50": float(t_pair[:, 1].median()),
            "step_us_p50": float(t_step.median()),
            "step_us_mean": float(t_step.mean()),
            "step_us_mean_with_mid_event": float(t_pair[:, 2].mean())}},
        "e2e_modes_us_per_step": modes,
        "e2e_note": graph_why,
        "h2d_bytes": arm.h2d_bytes(), "d2h_bytes": arm.d2h_bytes(),
        "wall_ms_per_step_incl_flush_and_barrier":
            (wall1 - wall0) * 1e3 / (2 * (h.steps + h.warmup)),
    }
    arm.close()
    if tokens != 1:
        one = Arm(kind, 1, rank, world, h.dev)
        t = h.time_pair(one.dispatch, one.combine, steps=min(h.steps, 100))
        one.close()
        res["latency_us"]["1"] = {"dispatch_us_p50": float(t[:, 0].median()),
                                  "combine_us_p50": float(t[:, 1].median()),
                                  "step_us_p50": float(t[:, 2].median())}
    return res


def e2e_entry(world: int, tokens: int, res: dict) -> dict:
    """The end-to-end entry of the JSON line.  Every mode is the whole step through the
    library's public API with the step's inputs starting in pinned host memory and its result
    ending there, inside the timed region; `value` is the best mode the library supports, the
    same rule for both arms, and all modes are listed."""
    modes = res["e2e_modes_us_per_step"]
    have = {k: v for k, v in modes.items() if v is not None}
    best = min(have, key=have.get)
    return {"value": world * tokens / (have[best] * 1e-6), "unit": "tokens/s",
            "us_per_step": have[best], "mode": best, "modes_us_per_step": modes,
            "h2d_bytes_per_step": res["h2d_bytes"], "d2h_bytes_per_step": res["d2h_bytes"],
            "note": res["e2e_note"]}


def config_entry(world: int, tokens: int, numa: str) -> dict:
    return {"model": "DeepSeek-V3 MoE layer all-to-all", "global_batch": world * tokens,
            "seq_len": 1, "tokens_per_gpu": tokens, "parallelism": f"ep{world}",
            "l2": "flushed between steps (256 MiB write)",
            "timing": "CUDA events around each step (dispatch + combine, nothing recorded in "
                      "between), ranks aligned by an NCCL all-reduce of one word before the first "
                      "event, max over ranks, mean over steps; dispatch/combine p50 from a second "
                      "pass with an event between the two",
            "host_placement": numa}


def vs_published(world: int, tokens: int, value: float) -> float | None:
    """value / the reference's published tokens/s; the published rows are EP8 only."""
    pub = PUBLISHED_US.get(tokens)
    if pub is None or world != PUBLISHED_WORLD:
        return None
    return value / (world * tokens / ((pub["dispatch"] + pub["combine"]) * 1e-6))


def base_line(world: int, tokens: int, steps: int, warmup: int, numa: str, res: dict) -> dict:
    main = res["latency_us"][str(tokens)]
    value = world * tokens / (main["step_us_mean"] * 1e-6)
    return {"metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": main["step_us_mean"] / 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": vs_published(world, tokens, value), "dtype": DTYPE,
            "data": DATA, "config": config_entry(world, tokens, numa),
            "latency_us": res["latency_us"],
            "published_reference_us": {str(k): v for k, v in PUBLISHED_US.items()},
            "published_reference_world": PUBLISHED_WORLD,
            "e2e": e2e_entry(world, tokens, res),
            "wall_ms_per_step_incl_flush_and_barrier":
                res["wall_ms_per_step_incl_flush_and_barrier"]}


def init_distributed(world: int, local_rank: int) -> None:
    if world > 1:
        torch.distributed.init_process_group(backend="cpu:gloo,cuda:nccl",
                                             device_id=torch.device("cuda", local_rank))
        try:
            torch._C._distributed_c10d._register_process_group("default",
                                                               torch.distributed.group.WORLD)
        except Exception:  # noqa: BLE001 - already registered
            pass


# ------------------------------------------------------------------ reference arm ----

def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        _emit({"impl": "reference", "unavailable": why})


def _reference_sub_arm(args: argparse.Namespace, kind: str) -> dict:
    """Measures one transport of the reference in this process."""
    rank, world, local_rank = _env_rank()
    dev = torch.device("cuda", local_rank)
    if kind == "ref-internode":
        # The path of the reference's own benchmark (tests/bench_all_to_all.py:60, 239-241):
        # NVSHMEM initialised from a unique id, then AllToAll.internode.
        import torch.distributed as dist
        from pplx_kernels import nvshmem as ref_nvshmem

        uid = (ref_nvshmem.nvshmem_get_unique_id() if rank == 0
               else ref_nvshmem.nvshmem_alloc_empty_unique_id())
        dist.broadcast(uid, src=0)
        ref_nvshmem.nvshmem_init(uid, rank, world)
    h = Harness(world, dev, args.steps, max(args.warmup, 3))
    res = measure_arm(kind, h, args.tokens, rank, world, args.no_graph)
    if kind == "ref-internode":
        ref_nvshmem.nvshmem_finalize()
    return res


def _internode_child(args: argparse.Namespace) -> dict:
    """Runs the NVSHMEM sub-arm in child processes (one per rank, started by every rank of the
    parent job) so that a failure or a hang of NVSHMEM's bring-up cannot take the parent's
    result with it.  Returns the child's result, or {"unavailable": reason}."""
    rank, world, local_rank = _env_rank()
    out_dir = os.environ.get("TMPDIR", tempfile.gettempdir())
    out_file = os.path.join(out_dir, f"pplx_ref_internode_{os.environ.get('MASTER_PORT', '0')}.json")
    if rank == 0 and os.path.exists(out_file):
        os.remove(out_file)
    torch.distributed.barrier()
    env = dict(os.environ)
    env["MASTER_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 23)
    # The children rendezvous among themselves: rank 0 of them hosts the store on the new port
    # (under torchrun the workers would otherwise look for the launcher's store there).
    env["TORCHELASTIC_USE_AGENT_STORE"] = "False"
    # The symmetric heap must hold the reference's buffers (about 1.9 GB at 128 tokens).
    env.setdefault("NVSHMEM_SYMMETRIC_SIZE", "6G")
    env.setdefault("NVSHMEM_REMOTE_TRANSPORT", "none")
    env.setdefault("NVSHMEM_DISABLE_CUDA_VMM", "0")
    cmd = [sys.executable, os.path.abspath(__file__), "--impl", "reference", "--ref-sub",
           "internode", "--out-file", out_file, "--gpus", str(world), "--steps", str(args.steps),
           "--warmup", str(args.warmup), "--tokens", str(args.tokens)]
    if args.no_graph:
        cmd.append("--no-graph")
    why = ""
    try:
        proc = subprocess.run(cmd, env=env, capture_output=True, text=True,
                              timeout=args.ref_child_timeout)
        if proc.returncode != 0:
            tail = (proc.stderr or proc.stdout or "").strip().splitlines()[-3:]
            why = f"exit code {proc.returncode}: " + " | ".join(tail)[-300:]
    except subprocess.TimeoutExpired:
        why = f"did not finish within {args.ref_child_timeout} s"
    ok = torch.tensor([0.0 if why else 1.0], device=torch.device("cuda", local_rank))
    torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
    reasons: list = [None] * world
    torch.distributed.all_gather_object(reasons, why)
    if ok.item() < 1.0:
        first = next((f"rank {r}: {w}" for r, w in enumerate(reasons) if w), "unknown")
        return {"unavailable": "AllToAll.internode over NVSHMEM (child processes): " + first}
    if rank != 0:
        return {}
    try:
        with open(out_file) as f:
            return json.load(f)
    except (OSError, ValueError) as exn:
        return {"unavailable": f"child result unreadable: {exn}"}


def reference_arm(args: argparse.Namespace) -> None:
    """The UNMODIFIED reference (installed under baseline/_ref by the offline pip command)
    through its own public API.  Two transports are measured with the harness of the other arm:
    ``AllToAll.intranode`` (its CUDA-IPC / NVLink kernels) in this process and
    ``AllToAll.internode`` (its NVSHMEM kernels over NVSHMEM's NVLink transport, the path its own
    benchmark uses) in child processes.  The faster one is the arm's `value`."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.exists(os.path.join(ref_dir, "pplx_kernels", "libpplx_kernels.so")):
        return _unavailable("baseline/_ref is empty: the offline install of the reference has "
                            "not been run on this machine")
    rank, world, local_rank = _env_rank()
    if world < 2:
        return _unavailable("the reference refuses a single rank: AllToAll.intranode asserts "
                            "world_size // dp_size > 1 (src/pplx_kernels/all_to_all.py:101)")
    sys.path.insert(0, ref_dir)
    from pplx_kernels_b200.parallel.affinity import bind_to_device_numa_node
    from pplx_kernels_b200.utils.clocks import ClockSampler

    torch.cuda.set_device(local_rank)
    numa = bind_to_device_numa_node(local_rank)  # same host placement in both arms
    init_distributed(world, local_rank)
    steps, warmup = args.steps, max(args.warmup, 3)

    if args.ref_sub == "internode":  # child process of _internode_child
        res = _reference_sub_arm(args, "ref-internode")
        if rank == 0:
            with open(args.out_file + ".tmp", "w") as f:
                json.dump(res, f)
            os.replace(args.out_file + ".tmp", args.out_file)
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
        return

    with ClockSampler(local_rank, period_ms=50) as sampler:
        intra = _reference_sub_arm(args, "ref-intranode")
    clocks = sampler.summary()
    inter = {"unavailable": "skipped (--ref-sub intranode)"}
    if args.ref_sub == "both":
        inter = _internode_child(args)

    def step_mean(res: dict) -> float:
        return res["latency_us"][str(args.tokens)]["step_us_mean"]

    best, best_name = intra, "AllToAll.intranode"
    if rank == 0 and "unavailable" not in inter and step_mean(inter) < step_mean(intra):
        best, best_name = inter, "AllToAll.internode"
    if rank == 0:
        line = base_line(world, args.tokens, steps, warmup, numa, best)
        line.update({
            "clocks": clocks, "gpu_launches": 2 * steps, "impl": "reference",
            "reference_path": f"pplx_kernels.{best_name} (unmodified, sm_100a build); the faster "
                              "of the two transports, both listed under sub_arms",
            "sub_arms": {"intranode": intra, "internode (NVSHMEM, NVLink transport)": inter},
            "repo_native_library_mapped": _repo_native_mapped(),
        })
        _emit(line)
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


# ------------------------------------------------------------------------ own arm ----

def nccl_baseline(h: Harness, cfg, tokens: int) -> float | None:
    """p50 microseconds of torch all_to_all_single on the reference's dense shape."""
    if h.world == 1:
        return None
    per_token = cfg.hidden_dim_bytes + cfg.hidden_dim_scale_bytes
    shape = (h.world, cfg.num_experts // h.world, tokens * per_token)
    src = torch.zeros(shape, dtype=torch.uint8, device=h.dev)
    dst = torch.empty_like(src)
    t = h.time_step(lambda: torch.distributed.all_to_all_single(dst, src), steps=min(h.steps, 50))
    return float(t.median())


def measured_nvlink_gbs(world: int) -> tuple[float, str]:
    """Peer-store bandwidth per direction seen by a plain copy kernel of the library (every
    rank stores 64 MiB into each peer at once), or the default when there is no peer."""
    if world < 2:
        return NVLINK_GBS_DEFAULT, "default (single GPU)"
    try:
        from pplx_kernels_b200.utils.peer_bandwidth import measure_peer_store_gbs

        return measure_peer_store_gbs(), "measured: all ranks store to all peers at once, copy kernel"
    except Exception as exn:  # noqa: BLE001 - the floor falls back to the default
        return NVLINK_GBS_DEFAULT, f"default ({type(exn).__name__}: {str(exn)[:80]})"


def own_arm(args: argparse.Namespace) -> None:
    rank, world, local_rank = _env_rank()
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from pplx_kernels_b200.parallel.affinity import bind_to_device_numa_node
    from pplx_kernels_b200.utils.clocks import ClockSampler

    numa = bind_to_device_numa_node(local_rank)  # before any pinned allocation
    init_distributed(world, local_rank)
    if world > 1:
        from pplx_kernels_b200.parallel.runtime import init_runtime_from_torch

        init_runtime_from_torch()
    steps, warmup = args.steps, max(args.warmup, 3)
    h = Harness(world, dev, steps, warmup)
    with ClockSampler(local_rank, period_ms=50) as sampler:
        res = measure_arm("ours", h, args.tokens, rank, world, args.no_graph)
    clocks = sampler.summary()
    from pplx_kernels_b200.utils.testing import DEEPSEEK_V3 as cfg

    nccl_us = nccl_baseline(h, cfg, args.tokens)
    res["latency_us"][str(args.tokens)]["nccl_all_to_all_single_us_p50"] = nccl_us
    link_gbs, link_how = measured_nvlink_gbs(world)

    # The second half of the headline metric: tokens/s of the whole MoE layer (dispatch ->
    # SwiGLU expert FFN on the tcgen05 grouped GEMM -> combine), Mixtral-8x7B shape, bf16.
    moe = None
    if not args.no_moe:
        from pplx_kernels_b200.utils.bench_moe import measure as measure_moe

        moe = measure_moe("mixtral-8x7b", 512, iters=10, warmup=3, rank=rank, world=world,
                          dev=dev, flush=h.flush)

    # Roofline of the headline step: bytes that must move over the slower path.
    peaks = _peaks()
    slot = cfg.hidden_dim_bytes + cfg.hidden_dim_scale_bytes + 16
    rows = args.tokens * cfg.experts_per_token
    disp_bytes = rows * slot
    comb_bytes = rows * cfg.hidden_dim * 2
    if world > 1:
        remote = (world - 1) / world
        floor_us = {"dispatch": disp_bytes * remote / NVLINK_GBS_DEFAULT / 1e3,
                    "combine": comb_bytes * remote / NVLINK_GBS_DEFAULT / 1e3}
        bound = (f"NVLink {NVLINK_GBS_DEFAULT:.0f} GB/s per direction (peer copy); this run's own "
                 f"copy kernel reached {link_gbs:.0f} GB/s ({link_how})")
    else:
        # single GPU: staging write + staging read + output write per row (dispatch);
        # staging write + staging read per row plus the token write (combine)
        hbm = float(peaks["hbm_gbs"])
        floor_us = {"dispatch": 3 * disp_bytes / hbm / 1e3, "combine": 2.125 * comb_bytes / hbm / 1e3}
        bound = f"HBM {hbm:.0f} GB/s of measured copy bandwidth"
    main_res = res["latency_us"][str(args.tokens)]
    roofline = {
        "bound": bound,
        "dispatch_floor_us": floor_us["dispatch"],
        "combine_floor_us": floor_us["combine"],
        "dispatch_frac": floor_us["dispatch"] / main_res["dispatch_us_p50"],
        "combine_frac": floor_us["combine"] / main_res["combine_us_p50"],
    }
    line = base_line(world, args.tokens, steps, warmup, numa, res)
    line.update({"roofline": roofline, "clocks": clocks, "gpu_launches": 2 * steps,
                 "moe_layer": moe, "impl": "ours"})
    if not args.no_moe:
        # The same layer in block-scaled fp8 with power-of-two scales, which the tensor cores
        # apply themselves (kind::mxf8f6f4.block_scale).  Informative only: neither an error nor
        # a rank that never comes back may cost the line above, so a timer prints the line
        # without this entry and ends the process if the measurement has not returned in time.
        import threading

        import pplx_kernels_b200.utils.bench_moe as bench_moe_mod

        def give_up() -> None:
            if rank == 0:
                line["moe_layer_fp8_hardware_scales"] = {"error": "did not finish in 180 s"}
                _emit(line)
            os._exit(0)

        timer = threading.Timer(180.0, give_up)
        timer.daemon = True
        timer.start()
        try:
            bench_moe_mod.POW2_SCALES = True
            moe_fp8 = measure_moe("mixtral-8x7b", 512, iters=10, warmup=3, rank=rank, world=world,
                                  dev=dev, flush=h.flush, fp8=True)
        except Exception as e:  # noqa: BLE001
            moe_fp8 = {"error": f"{type(e).__name__}: {e}"[:300]}
        finally:
            bench_moe_mod.POW2_SCALES = False
            timer.cancel()
        line["moe_layer_fp8_hardware_scales"] = moe_fp8
    if rank == 0:
        _emit(line)
    if world > 1:
        from pplx_kernels_b200.parallel.runtime import finalize_runtime

        torch.distributed.barrier()
        finalize_runtime()
        torch.distributed.destroy_process_group()


def sweep(args: argparse.Namespace) -> None:
    """One JSON line per (shape, tokens per GPU): dispatch / combine / step p50 of the chosen arm
    (max over ranks, L2 flushed, same harness as the headline run) and, in the own arm, torch's
    NCCL all_to_all_single on the reference's dense shape.  Serves the measurement tables."""
    rank, world, local_rank = _env_rank()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    init_distributed(world, local_rank)
    kind = "ours"
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        kind = "ref-internode" if args.ref_sub == "internode" else "ref-intranode"
        if kind == "ref-internode":
            from pplx_kernels import nvshmem as ref_nvshmem

            uid = (ref_nvshmem.nvshmem_get_unique_id() if rank == 0
                   else ref_nvshmem.nvshmem_alloc_empty_unique_id())
            torch.distributed.broadcast(uid, src=0)
            ref_nvshmem.nvshmem_init(uid, rank, world)
    h = Harness(world, dev, args.steps, max(args.warmup, 3))
    cases = [(shape, zipf, tokens) for shape in args.shapes.split(",")
             for zipf in (float(z) for z in str(args.zipf).split(","))
             for tokens in (int(t) for t in args.sweep.split(","))]
    for shape, zipf, tokens in cases:
        if SHAPES[shape][0] % world:
            continue
        arm = Arm(kind, tokens, rank, world, dev, shape=shape, zipf=zipf)
        t = h.time_pair(arm.dispatch, arm.combine)
        row = {"impl": kind, "shape": shape, "ep": world, "tokens": tokens, "zipf": zipf,
               "dispatch_us_p50": float(t[:, 0].median()),
               "combine_us_p50": float(t[:, 1].median()),
               "step_us_p50": float(t[:, 2].median()), "steps": h.steps}
        if kind == "ours":
            row["nccl_all_to_all_single_us_p50"] = (
                nccl_baseline(h, arm.cfg, tokens)
                if tokens * (arm.cfg.hidden_dim_bytes + arm.cfg.hidden_dim_scale_bytes)
                * arm.cfg.num_experts <= (2 << 30) else None)
            link = NVLINK_GBS_DEFAULT
            remote = (world - 1) / world
            rows = tokens * arm.cfg.experts_per_token
            slot = arm.cfg.hidden_dim_bytes + arm.cfg.hidden_dim_scale_bytes + 16
            if world > 1:
                row["dispatch_frac_of_nvlink_floor"] = (
                    rows * slot * remote / link / 1e3 / row["dispatch_us_p50"])
                row["combine_frac_of_nvlink_floor"] = (
                    rows * arm.cfg.hidden_dim * 2 * remote / link / 1e3 / row["combine_us_p50"])
        arm.close()
        if rank == 0:
            _emit(row)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--tokens", type=int, default=128, help="tokens per GPU of the headline run")
    ap.add_argument("--no-moe", action="store_true", help="skip the MoE-layer measurement")
    ap.add_argument("--no-graph", action="store_true",
                    help="skip the CUDA-graph replay of the end-to-end step")
    ap.add_argument("--ref-sub", choices=["both", "intranode", "internode"], default="both",
                    help="reference arm: which transport(s) to measure")
    ap.add_argument("--ref-child-timeout", type=int, default=300,
                    help="seconds the NVSHMEM sub-arm's child processes may take")
    ap.add_argument("--out-file", default="", help=argparse.SUPPRESS)
    ap.add_argument("--sweep", default="", help="comma list of tokens per GPU: print one JSON "
                    "line per size instead of the headline line")
    ap.add_argument("--shapes", default="r1", help="sweep: comma list of r1, v2lite")
    ap.add_argument("--zipf", default="0", help="sweep: routing skew(s), comma list; 0 = uniform")
    args = ap.parse_args()
    global _RESULT_FD
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    from pplx_kernels_b200.utils.logging_utils import init_logging

    init_logging()  # per-rank prefix on standard error; level from PPLX_B200_LOG_LEVEL
    if args.sweep:
        return sweep(args)
    if args.impl == "reference":
        try:
            reference_arm(args)
        except Exception as exn:  # the reference arm must never take the run down
            if args.ref_sub == "internode":
                raise
            _unavailable(f"reference run failed: {type(exn).__name__}: {str(exn)[:200]}")
        return
    own_arm(args)


if __name__ == "__main__":
    main()
