"""Benchmark of the YemongPolicy trunk hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C2|C2B|C3|C4|C5]

A step is one pass of the trunk over one batch of synthetic environments.  The default
workload is the full rollout policy step (all trunk attention layers + Griffin RG-LRU single
step with carried hidden state) at 4v4 + 4 refractive-field tokens = 12 tokens/env, 8192
envs, bf16 activations / fp32 state, random-init weights at the rl-fields profile's dims.
With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank runs its own
batch of that size: environments are independent, so there is no collective on the data
path, and the aggregate is N batches over the slowest rank's device time (weak scaling).

One JSON line is printed by rank 0: entity tokens/s with inputs resident in HBM (`value`),
the same through the public module API with pinned host buffers and both copies inside the
timed region (`e2e`), the HBM roofline fraction of the step from algorithmic bytes
(`roofline`), and the CPU oracle timed on the host cores on a bounded sample
(`cpu_baseline`).  `--impl reference` times that CPU restatement alone.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "policy-step entity tokens/sec per B200 (attn+RG-LRU), % of HBM roofline"
UNIT = "entity_tokens/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# DRAM bytes per entity token of the fused C2 step, from one ncu capture of k_trunk_pipelined on the
# half-size case (dram__bytes_read.sum + dram__bytes_write.sum = 310 730 496 B for 49 152 tokens,
# profiles/k_trunk_pipelined_c2_half.md); traffic grows in proportion to the tokens, so a full
# launch is this times its tokens.
NCU_C2_DRAM_BYTES_PER_TOKEN = (173093120 + 137637376) / 49152


def measured_peaks() -> tuple[float, float, float, str]:
    """(HBM GB/s, bf16 TFLOP/s burst, bf16 TFLOP/s sustained, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        burst = float(p["bf16_tflops"])
        return float(p["hbm_gbs"]), burst, float(p.get("bf16_tflops_sustained", burst)), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


def workloads_module():
    """The workload generators, loaded without running the package's __init__ (which would map
    libbnb_trunk.so into the process): the reference arm must not load the product."""
    if "boost_and_broadside_b200" in sys.modules:
        from boost_and_broadside_b200 import workloads as W

        return W
    import importlib
    import types

    if "_bnb_workloads" not in sys.modules:
        pkg = types.ModuleType("_bnb_workloads")
        pkg.__path__ = [os.path.join(ROOT, "boost-and-broadside_b200")]
        sys.modules["_bnb_workloads"] = pkg
    return importlib.import_module("_bnb_workloads.workloads")


def make_workload(name: str, rank: int, scale: float = 1.0):
    W = workloads_module()
    seed = 100 + rank
    if name == "C2":
        return W.c2(n_envs=max(1, int(8192 * scale)), seed=seed)
    if name == "C2B":
        return W.c2b(n_envs=max(1, int(8192 * scale)), seed=seed)
    if name == "C3":
        return W.c3(n_envs=max(1, int(1024 * scale)), seed=seed)
    if name == "C4":
        return W.c4(n_envs=max(1, int(4096 * scale)), seed=seed)
    if name == "C5":
        return W.c5(n_envs=max(1, int(16384 * scale)), seed=seed)
    raise SystemExit(f"unknown workload {name}")


WORKLOAD_TEXT = {
    "C2": "rollout trunk step, 8192 envs x (8 ships + 4 fields), bf16 activations / fp32 state",
    "C2B": "rollout trunk step with bullet cross-attention, 8192 envs x (8 ships + 4 fields + 80 bullet slots), bf16",
    "C3": "trunk step, 1024 envs x 152 ships (64 v 88), bf16",
    "C4": "recurrent-PPO sequence forward, T=32 x 4096 envs x 8 ships, bf16",
    "C5": "ragged trunk step, 16384 envs, tokens U{2..128}, bf16",
}


# ----------------------------------------------------------------------------- clocks


class ClockSampler:
    """SM clock and throttle-reason samples of one GPU during the timed region.

    The timed region of a default run lasts tens of milliseconds, shorter than the start-up of an
    `nvidia-smi -lms` process, so the samples are read through NVML (the library nvidia-smi itself
    uses) from a background thread every 2 ms; `nvidia-smi` is the fallback when the NVML binding is
    missing.  Only reads: no clock, power or mode setting is touched.
    """

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.file = None
        self.thread = None
        self.stop_flag = None
        self.sm, self.mx, self.reasons = [], [], set()
        self.source = None

    def _nvml_handle(self):
        import pynvml

        pynvml.nvmlInit()
        try:
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def start(self):
        try:
            import threading

            nv, handle = self._nvml_handle()
            max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.stop_flag = threading.Event()

            def loop():
                while not self.stop_flag.is_set():
                    try:
                        self.sm.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                        self.mx.append(max_mhz)
                        mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(handle))
                        for bit, name in self.REASONS.items():
                            if mask & bit:
                                self.reasons.add(name)
                    except Exception:
                        pass
                    time.sleep(0.002)

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            self.source = "nvml"
            return
        except Exception:
            self.thread = None
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.file, stderr=subprocess.DEVNULL)
            self.source = "nvidia-smi"
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": self.source}
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
        elif self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.file.flush()
            self.file.seek(0)
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for line in self.file.read().splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 7:
                    continue
                try:
                    self.sm.append(float(parts[0]))
                    self.mx.append(float(parts[1]))
                except ValueError:
                    continue
                for n, v in zip(names, parts[3:7]):
                    if v.lower().startswith("active"):
                        self.reasons.add(n)
            try:
                os.unlink(self.file.name)
            except OSError:
                pass
        if self.sm:
            out.update(sm_mhz=statistics.median(self.sm), sm_max_mhz=max(self.mx), reasons=sorted(self.reasons),
                       samples=len(self.sm))
        return out


# ----------------------------------------------------------------------------- CPU arm


def cpu_sample_scale(name: str) -> float:
    # bounded samples of the workload: about a second of CPU work per pass (C2: the full batch)
    return {"C2": 1.0, "C2B": 2048 / 8192, "C3": 128 / 1024, "C4": 128 / 4096, "C5": 2048 / 16384}[name]


def cpu_runner(name: str):
    """(callable, workload, kind, description) of the CPU arm: the reference's own modules from
    oracle/_ref when that copy exists (kind "reference"), else the oracle restatement ("port").
    Neither imports the product package."""
    from oracle import ref_runner

    w = make_workload(name, 0, cpu_sample_scale(name))
    if ref_runner.available():
        trunk = ref_runner.ReferenceTrunk().eval()
        return (ref_runner.workload_runner(trunk, w, "cpu"), w, "reference",
                "the reference's YemongBlock modules chained as models/yemong/policy.py:327-340 under "
                "torch.autocast('cpu', bfloat16)")
    from oracle import trunk_oracle as O

    # no copy of the reference on this machine: time the restatement, on weights of the layers' scale
    params = O.split_trunk_state_dict(O.synthetic_trunk_state_dict())
    if w.kind == "step":
        run = lambda: O.trunk_step(w.x, w.alive, w.hidden, params, 4, w.mode, w.bullets, w.bullet_mask)
    elif w.kind == "sequence":
        run = lambda: O.trunk_sequence(w.x, w.alive, w.hidden, w.done, params, 4, w.mode)
    else:
        nt, ns = w.n_tokens.tolist(), w.n_ships.tolist()
        run = lambda: O.trunk_step_ragged(w.x, w.alive, w.hidden, nt, ns, params, 4, w.mode)

    def run_no_grad():
        with torch.no_grad():
            return run()

    return run_no_grad, w, "port", "CPU restatement of the reference's forward (oracle/trunk_oracle.py)"


def time_cpu(name: str, passes: int, warmup: int) -> dict:
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    run, w, kind, what = cpu_runner(name)
    for _ in range(warmup):
        run()
    times = []
    for _ in range(passes):
        t0 = time.perf_counter()
        run()
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    return {
        "value": w.entity_tokens / t, "unit": UNIT, "cores": cores, "kind": kind,
        "sample": f"{w.meta.get('n_envs')} envs of {name} per pass ({w.entity_tokens} tokens), median of {passes} passes, "
                  f"{what}, {cores} threads",
        "ms_per_pass": t * 1e3, "tokens_per_pass": w.entity_tokens, "total_s": sum(times),
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    passes = max(1, min(args.steps, 30))
    warmup = max(0, min(args.warmup, 5))
    base = time_cpu(args.workload, passes, warmup)
    full = cpu_sample_scale(args.workload) == 1.0
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": passes, "warmup": warmup, "ms_per_step": base["ms_per_pass"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD_TEXT[args.workload], "id": args.workload,
                   "note": ("the reference's own PyTorch modules on the host cores, " +
                            ("the full batch per step" if full else "a bounded sample of the batch per step"))},
        "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- same-box GPU comparator


def time_gpu_reference(name: str, dev: torch.device, steps: int) -> dict:
    """The reference's own modules (oracle/_ref) on this GPU under torch.autocast('cuda', bfloat16),
    eager and as the reference runs them, torch.compile(mode="reduce-overhead")
    (train/rl/ppo.py:396-400 of the reference): the unfused library path the fused kernels replace.
    CUDA events over `steps` steps of the full workload."""
    from oracle import ref_runner

    out: dict = {}
    if not ref_runner.available():
        return {"unavailable": "oracle/_ref is absent"}
    w = make_workload(name, 0, 1.0)
    trunk = ref_runner.ReferenceTrunk().eval().to(dev)

    def timed(run, n):
        for _ in range(3):
            run()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            run()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / n

    try:
        run = ref_runner.workload_runner(trunk, w, str(dev))
        ms = timed(run, steps)
        out["eager"] = {"ms_per_step": ms, "value": w.entity_tokens / (ms * 1e-3), "unit": UNIT}
    except Exception as e:  # noqa: BLE001 - a comparator that fails is reported, not fatal
        out["eager"] = {"error": repr(e)[:200]}
    try:
        import copy

        compiled = copy.copy(trunk)
        compiled.step = torch.compile(trunk.step, mode="reduce-overhead")
        compiled.sequence = torch.compile(trunk.sequence, mode="reduce-overhead")
        run_c = ref_runner.workload_runner(compiled, w, str(dev))
        ms = timed(run_c, steps)
        out["compiled"] = {"ms_per_step": ms, "value": w.entity_tokens / (ms * 1e-3), "unit": UNIT,
                           "mode": "reduce-overhead"}
        if w.kind != "ragged":
            # with bfloat16 tokens, as its own encoder would hand them over: the reference then carries
            # the residual stream in bfloat16 too
            run_16 = ref_runner.workload_runner(compiled, w, str(dev), torch.bfloat16)
            ms = timed(run_16, steps)
            out["compiled_bf16_tokens"] = {"ms_per_step": ms, "value": w.entity_tokens / (ms * 1e-3), "unit": UNIT,
                                           "mode": "reduce-overhead"}
    except Exception as e:  # noqa: BLE001
        out.setdefault("compiled", {"error": repr(e)[:200]})
        out["compiled_error"] = repr(e)[:200]
    try:
        # the autocast contract of the encoders / heads (Linear -> RMSNorm) on this device
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            lin, norm = torch.nn.Linear(8, 8).to(dev), torch.nn.RMSNorm(8).to(dev)
            out["rmsnorm_after_linear_dtype"] = str(norm(lin(torch.zeros(2, 8, device=dev))).dtype)
    except Exception as e:  # noqa: BLE001
        out["rmsnorm_after_linear_dtype"] = repr(e)[:100]
    out["steps"] = steps
    out["what"] = "the reference's YemongBlock modules from oracle/_ref under torch.autocast('cuda', bfloat16), full workload"
    return out


def time_policy_step(dev: torch.device, n_envs: int = 8192, n_ships: int = 8, n_fields: int = 4, n_bullets: int = 80,
                     steps: int = 10, eager_only: bool = False) -> dict:
    """The whole rollout step of the policy, ``get_action_and_value`` (models/yemong/policy.py:291-373):
    FeatureCoordinator transforms, ship and bullet encoders, trunk step with bullets, the four heads,
    TeamPMA and the action draw, on one seeded random observation of `n_envs` environments under
    torch.autocast('cuda', bfloat16).  This package's YemongPolicy with the reference's state_dict
    loaded, against the reference's own policy from oracle/_ref, eager and torch.compile
    (mode="reduce-overhead", how the reference runs it: train/rl/ppo.py:396-400).  CUDA events."""
    from oracle import ref_runner

    if not ref_runner.available():
        return {"unavailable": "oracle/_ref is absent"}
    import boost_and_broadside_b200 as bnb
    from boost_and_broadside_b200 import _capi

    stock = ref_runner.reference_policy(n_ships).to(dev)
    cfg = bnb.ModelConfig(**ref_runner.RL_FIELDS)
    mine = bnb.YemongPolicy(cfg, stock.coordinator, num_value_components=11, num_ships=n_ships, team_pma_k=(0, 1),
                            bullet_coordinator=stock.bullet_encoder.coordinator).to(dev).eval()
    mine.load_state_dict(stock.state_dict(), strict=True)
    obs = ref_runner.random_observation(n_envs, n_ships, n_fields, n_bullets, seed=3, device=str(dev))
    hidden = torch.randn(mine.n_hidden_layers, n_envs * n_ships, 4 * cfg.d_model, device=dev) * 0.5

    def timed(fn):
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            for _ in range(3):
                fn()
            torch.cuda.synchronize(dev)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            before = _capi.lib.bnb_launch_count()
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            torch.cuda.synchronize(dev)
            return e0.elapsed_time(e1) / steps, (_capi.lib.bnb_launch_count() - before) / steps

    out: dict = {"workload": f"get_action_and_value, {n_envs} envs x ({n_ships} ships + {n_fields} fields), {n_bullets} bullet slots, "
                             "bf16 autocast", "env_steps_per_call": n_envs, "steps": steps}
    ms, launches = timed(lambda: mine.get_action_and_value(obs, hidden))
    out["ours"] = {"ms_per_step": ms, "env_steps_per_s": n_envs / (ms * 1e-3), "own_kernel_launches_per_step": launches}
    if eager_only:
        return out
    try:
        mine_c = torch.compile(mine.get_action_and_value, mode="reduce-overhead")
        ms, launches = timed(lambda: mine_c(obs, hidden))
        out["ours_compiled"] = {"ms_per_step": ms, "env_steps_per_s": n_envs / (ms * 1e-3), "mode": "reduce-overhead",
                                "note": "the same torch.compile call the reference makes: the FeatureCoordinator's torch operators are "
                                        "fused by the compiler, this package's kernels are opaque operators, and the step replays as "
                                        "one CUDA graph (own_kernel_launches_per_step counts host-side launch calls: 0 on replay)",
                                "own_kernel_launches_per_step": launches}
    except Exception as e:  # noqa: BLE001 - reported, not fatal
        out["ours_compiled"] = {"error": repr(e)[:300]}
    try:
        ms, _ = timed(lambda: stock.get_action_and_value(obs, hidden))
        out["reference_eager"] = {"ms_per_step": ms, "env_steps_per_s": n_envs / (ms * 1e-3)}
    except Exception as e:  # noqa: BLE001 - a comparator that fails is reported, not fatal
        out["reference_eager"] = {"error": repr(e)[:200]}
    try:
        compiled = torch.compile(stock.get_action_and_value, mode="reduce-overhead")
        ms, _ = timed(lambda: compiled(obs, hidden))
        out["reference_compiled"] = {"ms_per_step": ms, "env_steps_per_s": n_envs / (ms * 1e-3), "mode": "reduce-overhead"}
    except Exception as e:  # noqa: BLE001
        out["reference_compiled"] = {"error": repr(e)[:200]}
    return out


# ----------------------------------------------------------------------------- GPU arm


def time_train_step(trunk, dev: torch.device, n_envs: int = 1024, timesteps: int = 32, iters: int = 3,
                    with_reference: bool = True) -> dict:
    """Forward + backward of the sequence path at the PPO-update shape (C4's environments of 8 ships,
    T steps, bf16 autocast): loss = <y, dy>, gradients of tokens and every parameter.  This package
    (fused forward, bnb_trunk_sequence_bwd behind autograd) beside the reference's own modules from
    oracle/_ref through torch autograd, eager and torch.compile, same box, same shapes, CUDA events.
    The batch is a quarter of C4 because the reference's attention (cuDNN SDPA) refuses the full
    131072-environment-step batch when gradients are on."""
    from oracle import ref_runner

    W = workloads_module()
    w = W.c4(n_envs=n_envs, timesteps=timesteps)
    x, alive, hidden, done = (t.to(dev) for t in (w.x, w.alive, w.hidden, w.done))
    dy = torch.randn(x.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(0))
    tokens = w.entity_tokens
    out: dict = {"workload": f"C4 shape, {n_envs} environments x 8 ships x T={timesteps}, bf16 autocast, forward + backward",
                 "tokens_per_step": tokens, "iters": iters}

    def timed(fn):
        fn()
        torch.cuda.synchronize(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.reset_peak_memory_stats(dev)
        held = torch.cuda.memory_allocated(dev)   # tensors of the bench's other legs still alive: not this step's
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        ms = e0.elapsed_time(e1) / iters
        return {"ms_per_step": ms, "value": tokens / (ms * 1e-3), "unit": UNIT,
                "peak_gib": (torch.cuda.max_memory_allocated(dev) - held) / 2**30,
                "peak_note": "peak allocated during the timed steps above what was allocated before them "
                             "(inputs, parameters and kept gradients included in 'before')"}

    was_training = trunk.training
    trunk.train()

    def ours():
        trunk.zero_grad(set_to_none=True)
        xg = x.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            y, _ = trunk.sequence(xg, alive, hidden, done)
        (y.float() * dy).sum().backward()

    try:
        out["ours"] = timed(ours)
    finally:
        trunk.zero_grad(set_to_none=True)
        trunk.train(was_training)
    if not with_reference:
        return out
    if not ref_runner.available():
        out["reference"] = {"unavailable": "oracle/_ref is absent"}
        return out
    ref = ref_runner.ReferenceTrunk().train().to(dev)
    xb, ab, dyb = x.reshape(timesteps, n_envs, 8, -1), alive.reshape(timesteps, n_envs, 8), dy.reshape(timesteps, n_envs, 8, -1)

    def make(seq):
        def run():
            ref.zero_grad(set_to_none=True)
            xg = xb.clone().requires_grad_(True)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = seq(xg, ab, hidden, done)
            (y.float() * dyb).sum().backward()
        return run

    for key, seq in (("reference_eager", ref.sequence), ("reference_compiled", None)):
        try:
            if seq is None:
                seq = torch.compile(ref.sequence)
            out[key] = timed(make(seq))
            out[key]["ours_over_this"] = out["ours"]["value"] / out[key]["value"]
        except Exception as e:  # noqa: BLE001 - a comparator that fails is reported, not fatal
            out[key] = {"error": repr(e)[:200]}
    return out


def time_other_workloads(trunk, dev: torch.device, n_params_all: int, cfg, steps: int = 5) -> dict:
    """The other BASELINE configurations, device-timed like the headline (CUDA events, 3 warm-up
    steps, inputs resident, bf16 autocast, float32 tokens): C3 (152-token fleets), C4 (the T = 32
    sequence forward), C2B (C2 with 80 bullet slots per environment).  C5 is in c5_sharded."""
    W = workloads_module()
    hbm, tflops_burst, _, src = measured_peaks()
    out: dict = {}
    for name in ("C3", "C4", "C2B"):
        try:
            w = make_workload(name, 0, 1.0)
            x, alive, hidden = w.x.to(dev), w.alive.to(dev), w.hidden.to(dev)
            done = None if w.done is None else w.done.to(dev)
            bul = None if w.bullets is None else w.bullets.to(dev)
            bmask = None if w.bullet_mask is None else w.bullet_mask.to(dev)

            def run(h):
                if w.kind == "sequence":
                    return trunk.sequence(x, alive, h, done)
                return trunk.step(x, alive, h, bullets=bul, bullet_mask=bmask)

            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                h = hidden
                for _ in range(3):
                    _, h2 = run(h)
                    h = h if w.kind == "sequence" else h2
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(steps):
                    _, h2 = run(h)
                    h = h if w.kind == "sequence" else h2
                e1.record()
                torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1) / steps
            n_params = n_params_all if w.bullets is not None else sum(
                p.numel() for n, p in trunk.named_parameters() if "bullet" not in n)
            alg_bytes, alg_flops = W.algorithmic_bytes(w, n_params), W.algorithmic_flops(w, cfg)
            out[name] = {"workload": WORKLOAD_TEXT[name], "ms_per_step": ms, "value": w.entity_tokens / (ms * 1e-3), "unit": UNIT,
                         "steps": steps, "hbm_frac": alg_bytes / (ms * 1e-3) / 1e9 / hbm,
                         "tensor_frac_of_burst": alg_flops / (ms * 1e-3) / 1e12 / tflops_burst, "of": src}
            if w.kind != "sequence":
                # the same step with bfloat16 tokens (and bullet tokens), as the reference's encoders hand
                # them over under CUDA autocast: no float32 copies on either side of the kernels
                x, bul = x.to(torch.bfloat16), None if bul is None else bul.to(torch.bfloat16)
                with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                    for _ in range(3):
                        _, h = run(h)
                    torch.cuda.synchronize(dev)
                    e0.record()
                    for _ in range(steps):
                        _, h = run(h)
                    e1.record()
                    torch.cuda.synchronize(dev)
                ms16 = e0.elapsed_time(e1) / steps
                out[name]["bf16_tokens"] = {"ms_per_step": ms16, "value": w.entity_tokens / (ms16 * 1e-3), "unit": UNIT}
            del x, alive, hidden, h, h2, w
        except Exception as e:  # noqa: BLE001 - a side record that fails is reported, not fatal
            out[name] = {"error": repr(e)[:200]}
    return out


def run_train_only(args) -> None:
    """Only this package's forward + backward record, on one GPU (the command the launch-list
    profile of the training step is taken with)."""
    import boost_and_broadside_b200 as bnb

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    trunk = bnb.YemongTrunk(bnb.ModelConfig(d_model=128, n_heads=4, n_yemong_blocks=2, n_spatial_per_block=2,
                                            n_temporal_per_block=1, n_bullet_cross_per_block=1)).to(dev)
    print(json.dumps({"train_step": time_train_step(trunk, dev, n_envs=args.train_envs, iters=args.steps if args.steps < 20 else 3,
                                                    with_reference=False)}), flush=True)


def run_ours(args) -> None:
    import boost_and_broadside_b200 as bnb
    from boost_and_broadside_b200 import _capi
    from boost_and_broadside_b200 import workloads as W

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the trunk has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    if world > 1:
        # One process per GPU: run this rank on the CPUs next to its GPU, so that the pinned host
        # buffers of the end-to-end leg are placed (first touch) in that GPU's NUMA node instead of
        # all ranks sharing one socket's memory and the inter-socket link.
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(local).uuid)
            handle = pynvml.nvmlDeviceGetHandleByUUID((uuid if uuid.startswith("GPU-") else "GPU-" + uuid).encode())
            pynvml.nvmlDeviceSetCpuAffinity(handle)
        except Exception:
            pass

    cfg = W.rl_config()
    torch.manual_seed(0)
    trunk = bnb.YemongTrunk(cfg).eval()
    if args.shard and world > 1:
        from boost_and_broadside_b200 import sharding

        w = sharding.shard_workload(make_workload(args.workload, 0, args.envs_scale), rank, world)
    else:
        w = make_workload(args.workload, rank, args.envs_scale)
    n_params = sum(p.numel() for n, p in trunk.named_parameters() if w.bullets is not None or "bullet" not in n)
    trunk = trunk.to(dev)
    engine = {"auto": _capi.ENGINE_AUTO, "simt": _capi.ENGINE_SIMT, "tensor": _capi.ENGINE_TENSOR}[args.engine]

    x_h = w.x.pin_memory()
    alive_h = w.alive.pin_memory()
    x_d = x_h.to(dev, non_blocking=True)
    alive_d = alive_h.to(dev, non_blocking=True)
    hidden = [w.hidden.to(dev), None]
    done_d = None if w.done is None else w.done.to(dev)
    ragged = bnb.RaggedBatch(w.n_tokens, w.n_ships) if w.kind == "ragged" else None
    has_bullets = w.bullets is not None
    bul_h = w.bullets.pin_memory() if has_bullets else None
    bmask_h = w.bullet_mask.pin_memory() if has_bullets else None
    bul_d = bul_h.to(dev, non_blocking=True) if has_bullets else None
    bmask_d = bmask_h.to(dev, non_blocking=True) if has_bullets else None

    def step(xin, alive, h, bul=None, bmask=None):
        if w.kind == "step":
            if has_bullets:
                return trunk.step(xin, alive, h, engine=engine, bullets=bul_d if bul is None else bul,
                                  bullet_mask=bmask_d if bmask is None else bmask)
            return trunk.step(xin, alive, h, engine=engine)
        if w.kind == "sequence":
            return trunk.sequence(xin, alive, h, done_d, engine=engine)
        return trunk.step_ragged(xin, alive, h, ragged, engine=engine)

    carry = w.kind != "sequence"  # a sequence forward restarts from the same initial state
    ctx = torch.autocast("cuda", dtype=torch.bfloat16)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing
    with torch.no_grad(), ctx:
        h = hidden[0]
        for _ in range(args.warmup):
            y, h2 = step(x_d, alive_d, h)
            h = h2 if carry else h
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        launches0 = _capi.lib.bnb_launch_count()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        ev[0].record()
        for i in range(args.steps):
            y, h2 = step(x_d, alive_d, h)
            h = h2 if carry else h
            ev[i + 1].record()
        barrier()
        launches = _capi.lib.bnb_launch_count() - launches0
        clocks = sampler.stop() if rank == 0 else None
    total_ms = ev[0].elapsed_time(ev[-1])
    per_step = [ev[i].elapsed_time(ev[i + 1]) for i in range(args.steps)]

    # ---- end to end through the public API with pinned host buffers.  Every step copies its x and
    # alive from pinned host memory, runs the trunk, and copies y back to pinned host memory; the
    # three stages run on three streams so that step i+1's upload and step i-1's download overlap
    # step i's kernels (two device input buffers, two host output buffers).
    #
    # Token dtype of this leg: bfloat16 where the fused kernel takes it (C2, C4, C5) -- under
    # torch.autocast("cuda", bfloat16) the reference's encoder hands its trunk bfloat16 tokens and its
    # heads read the trunk's output as bfloat16 (see gpu_reference.rmsnorm_after_linear_dtype), so that
    # is the tensor a caller on the host side of this boundary holds; the module returns the dtype it
    # was given.  The same leg with float32 tokens is reported beside it as e2e_fp32_io.
    a_in = [torch.empty_like(alive_d) for _ in range(2)]
    b_in = [torch.empty_like(bul_d) for _ in range(2)] if has_bullets else None
    m_in = [torch.empty_like(bmask_d) for _ in range(2)] if has_bullets else None
    s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    # Three passes of K steps, the median pass reported: the host side of this leg (pinned memory,
    # PCIe root complex) is shared with the other tenants of the machine, and a single stall of theirs
    # inside a 20 ms pass would otherwise decide the figure.
    E2E_PASSES = 3

    def run_e2e(token_dtype):
        x_host = w.x.to(token_dtype).pin_memory()
        y_h = [torch.empty(w.x.shape, dtype=token_dtype).pin_memory() for _ in range(2)]
        x_in = [torch.empty(w.x.shape, dtype=token_dtype, device=dev) for _ in range(2)]
        y_stub = torch.empty(w.x.shape, dtype=token_dtype, device=dev)

        def e2e_loop(n, h, with_trunk=True):
            ev_in = [torch.cuda.Event() for _ in range(n)]
            ev_cmp = [torch.cuda.Event() for _ in range(n)]
            ev_out = [torch.cuda.Event() for _ in range(n)]
            for i in range(n):
                b = i % 2
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_cmp[i - 2])  # the kernels that read this input buffer are done
                    x_in[b].copy_(x_host, non_blocking=True)
                    a_in[b].copy_(alive_h, non_blocking=True)
                    if has_bullets:
                        b_in[b].copy_(bul_h, non_blocking=True)
                        m_in[b].copy_(bmask_h, non_blocking=True)
                    ev_in[i].record(s_in)
                with torch.cuda.stream(s_cmp):
                    s_cmp.wait_event(ev_in[i])
                    if with_trunk:
                        y, h2 = step(x_in[b], a_in[b], h, b_in[b] if has_bullets else None, m_in[b] if has_bullets else None)
                        h = h2 if carry else h
                    else:
                        y = y_stub   # the same copies without the kernels between them
                    ev_cmp[i].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[i])
                    if i >= 2:
                        s_out.wait_event(ev_out[i - 2])
                    y_h[b].copy_(y, non_blocking=True)
                    y.record_stream(s_out)
                    ev_out[i].record(s_out)
            return h

        times, copies = [], []
        with torch.no_grad(), ctx:
            h = hidden[0]
            h = e2e_loop(max(3, min(args.warmup, 5)), h)
            cur = torch.cuda.current_stream(dev)
            for with_trunk, sink in ((True, times), (False, copies)):
                for _ in range(E2E_PASSES):
                    barrier()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for st_ in (s_in, s_cmp, s_out):
                        st_.wait_event(e0)
                    h = e2e_loop(args.steps, h, with_trunk)
                    for st_ in (s_in, s_cmp, s_out):
                        cur.wait_stream(st_)
                    e1.record()
                    barrier()
                    sink.append(e0.elapsed_time(e1))
        assert y_h[0].dtype == token_dtype
        bytes_in = x_host.numel() * x_host.element_size() + alive_h.numel() + (bul_h.numel() * 4 + bmask_h.numel() if has_bullets else 0)
        bytes_out = y_h[0].numel() * y_h[0].element_size()
        return statistics.median(times), statistics.median(copies), times, bytes_in, bytes_out

    bf16_tokens = args.workload in ("C2", "C4", "C5") and args.engine != "simt"
    e2e_dtype = torch.bfloat16 if bf16_tokens else torch.float32
    e2e_ms, copy_ms, e2e_times, e2e_in, e2e_out = run_e2e(e2e_dtype)
    e2e32_ms, copy32_ms, _, e2e32_in, e2e32_out = run_e2e(torch.float32) if bf16_tokens else (e2e_ms, copy_ms, None, e2e_in, e2e_out)

    # ---- the ragged 16384-environment batch sharded contiguously over the ranks (strong scaling):
    # device-timed, max over ranks; one rank runs the whole batch.
    c5 = None
    if args.workload == "C2" and not args.no_c5:
        from boost_and_broadside_b200 import sharding

        w5 = make_workload("C5", 0, args.envs_scale)
        tokens5_all = w5.entity_tokens
        if world > 1:
            w5 = sharding.shard_workload(w5, rank, world)
        rb5 = bnb.RaggedBatch(w5.n_tokens, w5.n_ships)
        x5, a5, h5 = w5.x.to(dev), w5.alive.to(dev), w5.hidden.to(dev)
        n5 = max(3, min(args.steps, 10))
        with torch.no_grad(), ctx:
            for _ in range(3):
                _, h5n = trunk.step_ragged(x5, a5, h5, rb5, engine=engine)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(n5):
                _, h5n = trunk.step_ragged(x5, a5, h5, rb5, engine=engine)
            e1.record()
            barrier()
        t5 = torch.tensor([e0.elapsed_time(e1) / n5], dtype=torch.float64, device=dev)
        if dist is not None:
            dist.all_reduce(t5, op=dist.ReduceOp.MAX)
        c5 = {"workload": WORKLOAD_TEXT["C5"], "scaling": "strong", "ms_per_step": float(t5[0]),
              "value": tokens5_all / (float(t5[0]) * 1e-3), "unit": UNIT, "tokens_per_step": tokens5_all,
              "tokens_this_rank": w5.entity_tokens, "steps": n5,
              "note": "one global batch, environments sharded contiguously by rank, device-timed, max over ranks"}
        del x5, a5, h5, h5n

    t = torch.tensor([total_ms, e2e_ms, copy_ms, e2e32_ms, copy32_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, copy_ms, e2e32_ms, copy32_ms = (float(v) for v in t)
    tokens = w.entity_tokens
    if dist is not None:
        tk = torch.tensor([tokens], dtype=torch.float64, device=dev)
        dist.all_reduce(tk)
        tokens_all = float(tk[0])
    else:
        tokens_all = float(tokens)

    if rank == 0:
        hbm, tflops_burst, tflops, src = measured_peaks()
        ms_step = total_ms / args.steps
        alg_bytes = W.algorithmic_bytes(w, n_params)
        alg_flops = W.algorithmic_flops(w, cfg)
        kernel_ms = statistics.mean(per_step)
        achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": tokens_all * args.steps / (total_ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong" if args.shard and world > 1 else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": WORKLOAD_TEXT[args.workload], "id": args.workload, "engine": args.engine,
                       "tokens_per_step_per_gpu": tokens, "envs_scale": args.envs_scale, "l2": "inputs larger than L2 (no flush)",
                       "weights": "random init, seed 0, rl-fields dims (D=128, 4 heads, S S T | S S T)"},
            "e2e": {"value": tokens_all * args.steps / (e2e_ms * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": e2e_in, "d2h_bytes_per_step": e2e_out,
                    "token_dtype": str(e2e_dtype).replace("torch.", ""),
                    "note": "every step: x and alive from pinned host memory, trunk step through YemongTrunk, y back to pinned host "
                            "memory; upload, kernels and download pipelined on three streams; hidden state carried on the device; "
                            "median of 3 passes of K steps.  Tokens cross the boundary as " + str(e2e_dtype).replace("torch.", "") +
                            (": what the reference's trunk is handed and hands on under torch.autocast('cuda', bfloat16) "
                             "(gpu_reference.rmsnorm_after_linear_dtype); float32 tokens: e2e_fp32_io" if bf16_tokens else ""),
                    "passes_ms": [round(v, 3) for v in e2e_times],
                    "ms_per_step": e2e_ms / args.steps,
                    "copy_only_ms_per_step": copy_ms / args.steps,
                    "copy_only_note": "the same three-stream loop with the trunk call removed: the host-copy floor of this leg (max over ranks)"},
            "e2e_fp32_io": {"value": tokens_all * args.steps / (e2e32_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": e2e32_in,
                            "d2h_bytes_per_step": e2e32_out, "ms_per_step": e2e32_ms / args.steps,
                            "copy_only_ms_per_step": copy32_ms / args.steps,
                            "note": "the same leg with float32 tokens in and out (the dtype of last round's e2e)"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                         "traffic": (NCU_C2_DRAM_BYTES_PER_TOKEN * tokens if args.workload == "C2" and launches == 2 * args.steps else None),
                         "of": src, "algorithmic_bytes_per_step": alg_bytes,
                         "kernel": ("k_trunk_pipelined (one launch = one trunk step; the 8 us k_pack_trunk launch that rewrites the weight images before it is inside the timed step)"
                                    if launches == 2 * args.steps else "whole trunk step (all launches of one step)"), "kernel_ms": kernel_ms},
            "tensor": {"achieved": alg_flops / (kernel_ms * 1e-3) / 1e12, "peak": tflops_burst, "unit": "TFLOP/s",
                       "frac": alg_flops / (kernel_ms * 1e-3) / 1e12 / tflops_burst, "of": src + " (burst: the timed region lasts milliseconds)",
                       "frac_of_sustained": alg_flops / (kernel_ms * 1e-3) / 1e12 / tflops, "peak_sustained": tflops,
                       "algorithmic_flops_per_step": alg_flops},
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons", "samples", "source")} if clocks else None,
        }
        if c5 is not None:
            line["c5_sharded"] = c5
        if world == 1 and not args.no_gpu_ref:
            ref = time_gpu_reference(args.workload, dev, 20)
            for k in ("eager", "compiled", "compiled_bf16_tokens"):
                if isinstance(ref.get(k), dict) and "value" in ref[k]:
                    ref[k]["ours_over_this"] = line["value"] / ref[k]["value"]
            line["gpu_reference"] = ref
        if world == 1 and not args.no_others and args.workload == "C2":
            line["other_workloads"] = time_other_workloads(
                trunk, dev, sum(p.numel() for p in trunk.parameters()), cfg)
        if world == 1 and not args.no_train and args.workload == "C2":
            line["train_step"] = time_train_step(trunk, dev)
        if world == 1 and not args.no_policy and args.workload == "C2":
            line["policy_step"] = time_policy_step(dev)
        if world == 1 and not args.no_cpu:
            base = time_cpu(args.workload, 3, 1)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOAD_TEXT))
    ap.add_argument("--engine", default="auto", choices=["auto", "simt", "tensor"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--no-gpu-ref", action="store_true", help="skip the same-box GPU comparator (reference modules, eager and compiled)")
    ap.add_argument("--no-c5", action="store_true", help="skip the sharded ragged C5 record")
    ap.add_argument("--no-train", action="store_true", help="skip the forward + backward record (train_step)")
    ap.add_argument("--no-policy", action="store_true", help="skip the whole-policy rollout step record (policy_step)")
    ap.add_argument("--policy-only", action="store_true", help="only the whole-policy rollout step record (for profiling)")
    ap.add_argument("--policy-eager", action="store_true", help="with --policy-only: this package's eager leg alone (for profiler captures)")
    ap.add_argument("--no-others", action="store_true", help="skip the C3 / C4 / C2B records (other_workloads)")
    ap.add_argument("--train-only", action="store_true", help="only this package's forward + backward record (for profiling)")
    ap.add_argument("--train-envs", type=int, default=1024, help="environments of the forward + backward record")
    ap.add_argument("--shard", action="store_true",
                    help="one global batch, environments sharded contiguously over the ranks (strong scaling) "
                         "instead of one full batch per rank")
    ap.add_argument("--envs-scale", type=float, default=1.0,
                    help="fraction of the workload's environments (small cases for profiler captures only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.train_only:
        run_train_only(args)
    elif args.policy_only:
        torch.cuda.set_device(0)
        print(json.dumps({"policy_step": time_policy_step(torch.device("cuda", 0), steps=args.steps if args.steps < 20 else 10,
                                                          eager_only=args.policy_eager)}), flush=True)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
