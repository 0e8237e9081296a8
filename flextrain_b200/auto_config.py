"""One-shot profiler + LP planner for the offload ratios.

Parity: flextrain/auto_config.py:1-688 - ``system_auto_config`` :58-346
(micro-benchmarks of layer forward/backward, PCIe, NVMe and the host Adam,
20-80 percentile means averaged over ranks), ``MachinePerfParams`` :349-378,
``ConfigResult`` :381-389 and ``FlexTrainConfigSolver`` :392-688 (enumerate
micro-batches per rank and alpha, solve an LP for the split ratios, stop when
throughput stops improving, print the candidates).

What differs, on purpose
  * HBM is a tier: the LP has ``gpu_para``, ``gpu_opts`` and ``gpu_ckpt``
    variables (the reference asserts those shares to zero), a device-Adam rate
    and an NVLink term for the gather / reduce-scatter;
  * the LP is solved by ``flextrain_b200.lp`` (SciPy's HiGHS or the in-repo
    simplex), there is no PuLP dependency;
  * the planner returns its candidates (and logs them) instead of calling
    ``exit()``; ``engine.train_iteration`` keeps running with the current config.
"""
from __future__ import annotations

import os
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import torch

from . import defaults as D
from .lp import LinearProgram
from .utils import distributed as dist
from .utils.logging import rank0_logger


# ------------------------------------------------------------------ helpers
def trimmed_mean(samples: List[float]) -> float:
    """Mean of the 20th..80th percentile band (flextrain/auto_config.py:48-55)."""
    s = sorted(samples)
    lo, hi = int(len(s) * 0.2), max(int(len(s) * 0.8), int(len(s) * 0.2) + 1)
    band = s[lo:hi]
    return sum(band) / len(band)


def world_mean(value: float) -> float:
    return dist.all_reduce_scalar(value) / dist.get_world_size()


@dataclass
class MachinePerfParams:
    world_size: int
    num_layers: int                 # units
    opt_states: int                 # optimizer states per element (2 for Adam)
    device_itemsize: int
    gradacc_itemsize: int
    master_itemsize: int
    layer_fwd_time: float           # s per micro-batch per unit
    layer_bwd_time: float
    pre_post_time: float            # s per micro-batch (pre + post + loss, fwd + bwd)
    vram_bytes: float               # usable HBM per rank, working set already deducted
    dram_bytes: float               # usable host DRAM per rank
    nvme_bytes: float               # usable NVMe per rank
    unit_numel: int                 # aligned unit numel (whole unit, all ranks)
    interlayer_numel: int           # inter-unit activation numel per micro-batch
    pcie_bandwidth: float           # B/s per rank, one direction
    nvme_read_bandwidth: float      # B/s per rank
    nvme_write_bandwidth: float
    cpu_adam_throughput: float      # elements/s per rank
    gpu_adam_throughput: float      # elements/s per rank
    nvlink_bandwidth: float         # B/s per rank, one direction
    pcie_h2d_bandwidth: float = 0.0  # B/s per rank, host to device (0: take pcie_bandwidth)
    nvme_backend: str = ""          # which backend the NVMe engine was granted (io_uring, ...)


@dataclass
class ConfigResult:
    micro_batches_per_rank: int
    alpha: float
    throughput: float               # micro-batches / s, whole job
    iteration_time: float
    split_ratio: Dict[str, List[float]] = field(default_factory=dict)

    def to_config(self) -> Dict:
        return {"split_ratio": {**self.split_ratio, "alpha": self.alpha}}


class FlexTrainConfigSolver:
    """Enumerates ``(micro_batches_per_rank, alpha)`` and solves one LP each."""

    def __init__(self, perf: MachinePerfParams, alphas: Optional[List[float]] = None,
                 max_mbpr: int = 64):
        self.p = perf
        self.alphas = alphas if alphas is not None else D.POTENTIAL_ALPHA_VALUES[::5]
        self.max_mbpr = max_mbpr

    # ------------------------------------------------------------------ LP
    def _solve_given_hypers(self, mbpr: int, alpha: float) -> Optional[ConfigResult]:
        p = self.p
        W, L, S = p.world_size, p.num_layers, p.opt_states
        d, g, m = p.device_itemsize, p.gradacc_itemsize, p.master_itemsize
        P = p.unit_numel / W                  # elements of one unit owned by this rank
        A = p.interlayer_numel
        lp = LinearProgram()
        v = {}
        for kind in ("ckpt", "para", "opts"):
            for tier in ("gpu", "cpu", "nvme"):
                v[f"{tier}_{kind}"] = lp.var(f"{tier}_{kind}", 0.0, 1.0)
            lp.add_eq({f"gpu_{kind}": 1, f"cpu_{kind}": 1, f"nvme_{kind}": 1}, 1.0)
        lp.var("gpu_grad", 0.0, 1.0)
        lp.var("cpu_grad", 0.0, 1.0)
        lp.add_eq({"gpu_grad": 1, "cpu_grad": 1}, 1.0)
        lp.var("T_f", 0.0, None)
        lp.var("T_b", 0.0, None)
        # Among placements of equal step time (a compute-bound step leaves the LP indifferent)
        # prefer the nearer tier for every kind of data: a whole share in NVMe is charged a tenth of
        # a layer's forward time, a whole share in host memory a fiftieth.
        far, near = 10 * D.REGULARIZATION_PENALTY * p.layer_fwd_time, 2 * D.REGULARIZATION_PENALTY * p.layer_fwd_time
        lp.minimise({"T_f": 1.0, "T_b": 1.0,
                     "nvme_para": far, "nvme_opts": far, "nvme_ckpt": far,
                     "cpu_opts": near, "cpu_para": near, "cpu_ckpt": near, "cpu_grad": near})
        opt_bytes = P * m * (S + 1)
        # ---- capacity
        lp.add_le({"gpu_para": P * L * d, "gpu_opts": opt_bytes * L, "gpu_ckpt": mbpr * A * L * d,
                   "gpu_grad": mbpr * A * d}, p.vram_bytes)
        host_staging = (2 + alpha * L) * P * g                       # pinned gradient pool
        lp.add_le({"cpu_para": P * L * d, "cpu_opts": opt_bytes * L, "cpu_ckpt": mbpr * A * L * d,
                   "cpu_grad": mbpr * A * d, "nvme_opts": opt_bytes, "nvme_para": 2 * P * d,
                   "nvme_ckpt": 2 * A * d}, max(p.dram_bytes - host_staging, 0.0))
        lp.add_le({"nvme_para": P * L * d, "nvme_opts": opt_bytes * L, "nvme_ckpt": mbpr * A * L * d},
                  p.nvme_bytes)
        # ---- compute
        lp.add_ge({"T_f": 1.0}, p.layer_fwd_time * mbpr)
        lp.add_ge({"T_b": 1.0}, (p.layer_fwd_time + p.layer_bwd_time) * mbpr)
        # ---- optimizer throughput (host share may spill alpha of its work into forward)
        host = {"cpu_opts": P, "nvme_opts": P}
        lp.add_le({**{k: c * (1 - alpha) for k, c in host.items()}, "T_b": -p.cpu_adam_throughput}, 0.0)
        lp.add_le({**{k: c * alpha for k, c in host.items()}, "T_f": -p.cpu_adam_throughput}, 0.0)
        lp.add_le({"gpu_opts": P, "T_b": -p.gpu_adam_throughput}, 0.0)
        # ---- PCIe, per direction
        bw = p.pcie_bandwidth
        bw_in = p.pcie_h2d_bandwidth if p.pcie_h2d_bandwidth > 0 else bw
        h2d_f = {"cpu_para": P * d, "nvme_para": P * d}
        d2h_f = {"cpu_ckpt": mbpr * A * d, "nvme_ckpt": mbpr * A * d}
        lp.add_le({**h2d_f, "T_f": -bw_in}, 0.0)
        lp.add_le({**d2h_f, "T_f": -bw}, 0.0)
        h2d_b = {"cpu_para": P * d, "nvme_para": P * d, "cpu_ckpt": mbpr * A * d,
                 "nvme_ckpt": mbpr * A * d, "cpu_grad": mbpr * A * d}
        d2h_b = {"cpu_opts": P * g, "nvme_opts": P * g, "cpu_grad": mbpr * A * d}
        lp.add_le({**h2d_b, "T_b": -bw_in}, 0.0)
        lp.add_le({**d2h_b, "T_b": -bw}, 0.0)
        # ---- NVMe (read + write share the device)
        rd, wr = p.nvme_read_bandwidth, p.nvme_write_bandwidth
        if rd > 0 and wr > 0:
            lp.add_le({"nvme_para": P * d / rd, "nvme_ckpt": mbpr * A * d / wr,
                       "nvme_opts": alpha * opt_bytes * (1 / rd + 1 / wr), "T_f": -1.0}, 0.0)
            lp.add_le({"nvme_para": P * d * (1 / rd + 1 / wr), "nvme_ckpt": mbpr * A * d / rd,
                       "nvme_opts": (1 - alpha) * opt_bytes * (1 / rd + 1 / wr), "T_b": -1.0}, 0.0)
        else:
            lp.add_le({"nvme_para": 1.0, "nvme_opts": 1.0, "nvme_ckpt": 1.0}, 0.0)
        # ---- NVLink: gather in forward and backward, reduce-scatter in backward
        if W > 1 and p.nvlink_bandwidth > 0:
            link = P * (W - 1)
            lp.add_ge({"T_f": p.nvlink_bandwidth}, link * d)
            lp.add_ge({"T_b": p.nvlink_bandwidth}, link * d + link * g)
        sol = lp.solve()
        if sol is None:
            return None
        iter_time = (sol["T_f"] + sol["T_b"]) * L + p.pre_post_time * mbpr
        ratios = {
            "checkpoint": [round(sol["gpu_ckpt"], 4), round(sol["cpu_ckpt"], 4)],
            "parameter": [round(sol["gpu_para"], 4), round(sol["cpu_para"], 4)],
            "optimizer": [round(sol["gpu_opts"], 4), round(sol["cpu_opts"], 4)],
            "gradient": [round(sol["gpu_grad"], 4), round(1 - round(sol["gpu_grad"], 4), 4)],
        }
        for k in ("checkpoint", "parameter", "optimizer"):
            gsh, csh = ratios[k]
            if gsh + csh > 1.0:
                ratios[k] = [gsh, round(1.0 - gsh, 4)]
        return ConfigResult(mbpr, alpha, mbpr * W / iter_time, iter_time, ratios)

    # ------------------------------------------------------------ enumerate
    def solve(self) -> List[ConfigResult]:
        """Best result per ``mbpr`` (an alpha is preferred only if it is >= 1 %
        faster), stopping ``NUM_EXTRA_CONFIGS`` values after the throughput
        stopped improving (flextrain/auto_config.py:428-469)."""
        results: List[ConfigResult] = []
        best, since_best = 0.0, 0
        for mbpr in range(1, self.max_mbpr + 1):
            chosen: Optional[ConfigResult] = None
            for alpha in self.alphas:
                r = self._solve_given_hypers(mbpr, alpha)
                if r is None:
                    continue
                if chosen is None or r.throughput > chosen.throughput * D.THROUGHPUT_STABLE_THRESHOLD:
                    chosen = r
            if chosen is None:
                if results:
                    break
                continue
            results.append(chosen)
            if chosen.throughput > best * D.THROUGHPUT_STABLE_THRESHOLD:
                best, since_best = chosen.throughput, 0
            else:
                since_best += 1
                if since_best >= D.NUM_EXTRA_CONFIGS:
                    break
        return results


def format_results(results: List[ConfigResult]) -> str:
    lines = ["auto-config candidates (best alpha per micro-batch count):"]
    for r in results:
        lines.append(f"  mbpr={r.micro_batches_per_rank:3d} alpha={r.alpha:.2f} "
                     f"throughput={r.throughput:8.3f} micro-batch/s iter={r.iteration_time * 1e3:9.1f} ms "
                     f"ratios={r.split_ratio}")
    return "\n".join(lines)


# --------------------------------------------------------------- profiling
def _time_cuda(fn, iters: int) -> float:
    samples = []
    for _ in range(iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        e.synchronize()
        samples.append(s.elapsed_time(e) / 1e3)
    return trimmed_mean(samples)


def _time_host(fn, iters: int) -> float:
    samples = []
    for _ in range(iters):
        t0 = time.perf_counter()
        fn()
        samples.append(time.perf_counter() - t0)
    return trimmed_mean(samples)


def benchmark_pcie(device, nbytes: int = 1 << 28, iters: int = 20, h2d: bool = False) -> float:
    """Bandwidth of a pinned copy, B/s: device to host, or host to device with ``h2d``."""
    if device.type != "cuda":
        return 50e9
    from .memory import allocate_memory
    host = allocate_memory(nbytes, torch.uint8, "cpu", True)
    dev = torch.empty(nbytes, dtype=torch.uint8, device=device)
    host.copy_(dev)
    torch.cuda.synchronize()
    if h2d:
        t = _time_cuda(lambda: dev.copy_(host, non_blocking=True), iters)
    else:
        t = _time_cuda(lambda: host.copy_(dev, non_blocking=True), iters)
    return nbytes / t


def benchmark_nvme(swap_dir: str, nbytes: int = 1 << 30, iters: int = 3):
    """(read B/s, write B/s) of the NVMe engine on ``swap_dir``; (0, 0) if unusable.  The
    transfers are large (1 GiB each, like a unit's optimizer state) because what the planner
    needs is the rate the device sustains, not what a cache in front of it absorbs."""
    from .memory.nvme_swapper import NVMeEngine
    try:
        os.makedirs(swap_dir, exist_ok=True)
        eng = NVMeEngine()
        buf = torch.empty(nbytes, dtype=torch.uint8)
        path = os.path.join(swap_dir, f"rank{dist.get_rank()}_BENCH.swp")
        tw = _time_host(lambda: eng.write(path, buf), iters)
        tr = _time_host(lambda: eng.read(path, buf), iters)
        eng.forget(path)
        os.remove(path)
        eng.close()
        return nbytes / tr, nbytes / tw
    except Exception as exc:
        rank0_logger.warning(f"NVMe benchmark failed ({exc}); the planner will not use NVMe")
        return 0.0, 0.0


def benchmark_cpu_adam(cpu_optimizer, device_dtype, numel: int = 1 << 24, iters: int = 8) -> float:
    cpu_optimizer.profile_step(numel, device_dtype, torch.float32)
    t = trimmed_mean([cpu_optimizer.profile_step(numel, device_dtype, torch.float32)
                      for _ in range(iters)])
    return numel / t


def benchmark_gpu_adam(device, device_dtype, owner, numel: int = 1 << 26, iters: int = 10) -> float:
    if device.type != "cuda":
        return 5e9
    from .ops.adam.gpu_adam import device_adam_update
    p = torch.randn(numel, device=device)
    g = torch.randn(numel, device=device).to(device_dtype)
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    out = torch.empty(numel, device=device, dtype=device_dtype)
    fn = lambda: device_adam_update({}, 1, owner, p, g, [m, v], out)  # noqa: E731
    fn()
    return numel / _time_cuda(fn, iters)


def benchmark_nvlink(device, nbytes: int = 1 << 28, iters: int = 10) -> float:
    """All-gather bandwidth per rank (bytes received / s); 0 when alone."""
    world = dist.get_world_size()
    if world == 1 or device.type != "cuda":
        return 0.0
    shard = torch.empty(nbytes // world, dtype=torch.uint8, device=device)
    full = torch.empty(nbytes // world * world, dtype=torch.uint8, device=device)
    dist.all_gather(full, shard)
    t = _time_cuda(lambda: dist.all_gather(full, shard), iters)
    return shard.numel() * (world - 1) / t


def benchmark_layers(engine, iters: int = 10):
    """(layer fwd s, layer bwd s, pre+post s) for one micro-batch, measured with
    the registered callbacks on unit 0."""
    from .llm_func import LLMFunc, retrieve_llm_loss
    para = engine.para
    cuda = engine.device.type == "cuda"
    timer = _time_cuda if cuda else _time_host
    para.acquire(0)
    start, end = engine._layer_range(0)
    pre, post, loss_in = LLMFunc.get_batch()
    with torch.no_grad():
        passed, every = LLMFunc.pre_process(pre)
    passed = tuple(t.detach() if torch.is_tensor(t) else t for t in passed)
    layer = LLMFunc.layer_forward(start, end)

    def fwd():
        with torch.no_grad():
            layer(*passed, *every)

    def fwd_bwd():
        inp = tuple(t.detach().requires_grad_() if torch.is_tensor(t) and t.is_floating_point() else t
                    for t in passed)
        out = layer(*inp, *every)
        out = out[0] if isinstance(out, (tuple, list)) else out
        out.backward(torch.ones_like(out))

    def pre_post():
        p2, e2 = LLMFunc.pre_process(pre)
        outs = LLMFunc.post_process(p2, post)
        retrieve_llm_loss(LLMFunc.loss(outs, loss_in)).float().backward()

    grads_before = [p.grad for p in para.unit_group(0).paras]
    fwd()
    t_f = timer(fwd, iters)
    fwd_bwd()
    t_fb = timer(fwd_bwd, iters)
    pre_post()
    t_pp = timer(pre_post, max(2, iters // 3))
    for p, g0 in zip(para.unit_group(0).paras, grads_before):
        p.grad = g0
    for p in engine.optimizer.non_layerwise_params:
        if p.grad is not None:
            p.grad.zero_()
    para.release(0)
    return t_f / engine.interval, max(t_fb - t_f, t_f) / engine.interval, t_pp


def measure_machine(engine, iters: int = 10, swap_dir: Optional[str] = None) -> MachinePerfParams:
    import psutil
    cfg = engine.config
    mp = cfg.mixed_precision
    dev = engine.device
    t_f, t_b, t_pp = benchmark_layers(engine, iters)
    itemsize = lambda dt: torch.empty((), dtype=dt).element_size()  # noqa: E731
    if dev.type == "cuda":
        # what the driver reports free plus what the current placement spends on movable state;
        # blocks cached by the allocator are the step's working set and stay out of the budget
        free, _total = torch.cuda.mem_get_info()
        vram = (free + _tier_bytes(engine, "hbm")) * D.ACCESSIBLE_GPU_MEMORY_RATIO
    else:
        vram = 8e9
    dram = min(cfg.max_dram_usage * 1e9 if cfg.max_dram_usage > 0 else float("inf"),
               (psutil.virtual_memory().available + _tier_bytes(engine, "dram"))
               * D.ACCESSIBLE_CPU_MEMORY_RATIO) / dist.get_world_size()
    swap_dir = swap_dir or cfg.nvme_swap.swap_dir
    nv_r, nv_w = benchmark_nvme(swap_dir)
    try:
        import shutil
        nvme_free = shutil.disk_usage(swap_dir).free * 0.9 / dist.get_world_size()
    except OSError:
        nvme_free = 0.0
    A = engine.inter.ckpt._numel or 0
    perf = MachinePerfParams(
        world_size=dist.get_world_size(), num_layers=engine.num_units,
        opt_states=engine.optimizer.optimizer_state_per_element,
        device_itemsize=itemsize(mp.device_dtype), gradacc_itemsize=itemsize(mp.gradacc_dtype),
        master_itemsize=itemsize(mp.master_dtype),
        layer_fwd_time=world_mean(t_f) * engine.interval, layer_bwd_time=world_mean(t_b) * engine.interval,
        pre_post_time=world_mean(t_pp), vram_bytes=vram, dram_bytes=dram, nvme_bytes=nvme_free,
        unit_numel=engine.para.aligned_unit_numel, interlayer_numel=A,
        pcie_bandwidth=world_mean(benchmark_pcie(dev)), nvme_read_bandwidth=world_mean(nv_r),
        nvme_write_bandwidth=world_mean(nv_w),
        cpu_adam_throughput=world_mean(benchmark_cpu_adam(engine.optimizer.cpu_optimizer, mp.device_dtype)),
        gpu_adam_throughput=world_mean(benchmark_gpu_adam(dev, mp.device_dtype,
                                                          engine.optimizer.cpu_optimizer)),
        nvlink_bandwidth=world_mean(benchmark_nvlink(dev)),
        pcie_h2d_bandwidth=world_mean(benchmark_pcie(dev, h2d=True)),
        nvme_backend=_nvme_backend_name())
    return perf


def _nvme_backend_name() -> str:
    try:
        from .memory.nvme_swapper import NVMeEngine
        eng = NVMeEngine()
        name = str(eng.kind)
        eng.close()
        return name
    except Exception:
        return "unknown"


def _tier_bytes(engine, kind: str) -> float:
    """Bytes the current config already spends on movable state in ``kind``
    (they become available again once the planner re-places them)."""
    para, opts = engine.para, engine.opts
    isz = para.itemsize
    if kind == "hbm":
        return para.tier_numels[0] * isz * para.num_units + opts.opt_tiers[0] * 4 * opts.K * para.num_units
    return para.tier_numels[1] * isz * para.num_units + opts.opt_tiers[1] * 4 * opts.K * para.num_units


def system_auto_config(engine, iters: int = 10) -> List[ConfigResult]:
    """Profile the machine with the live engine, solve the planner and log the
    candidates.  Returns them (best first by throughput)."""
    engine.synchronize()
    perf = measure_machine(engine, iters)
    rank0_logger.info("auto-config measurements:\n" +
                      "\n".join(f"  {k} = {v:.6g}" if isinstance(v, float) else f"  {k} = {v}"
                                for k, v in asdict(perf).items()))
    results = FlexTrainConfigSolver(perf).solve() if dist.get_rank() == 0 else []
    if dist.get_rank() == 0:
        rank0_logger.info(format_results(results))
    engine.last_auto_config = results
    # best first; within 1 % of each other the smaller batch (less memory, same rate) comes first
    top = max((r.throughput for r in results), default=0.0)
    results = sorted(results, key=lambda r: (0 if r.throughput >= top / D.THROUGHPUT_STABLE_THRESHOLD else 1,
                                             r.micro_batches_per_rank if r.throughput >= top / D.THROUGHPUT_STABLE_THRESHOLD
                                             else -r.throughput))
    engine.auto_config_report = {
        "measurements": asdict(perf),
        "candidates": [{"micro_batches_per_rank": r.micro_batches_per_rank, "alpha": r.alpha,
                        "predicted_micro_batches_per_s": r.throughput,
                        "predicted_iteration_ms": r.iteration_time * 1e3,
                        "split_ratio": {**r.split_ratio, "alpha": r.alpha}} for r in results[:6]]}
    return results
