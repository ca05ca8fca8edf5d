"""Benchmark of the block-Gibbs hot path.

    python bench.py --gpus N --steps K --warmup W                      # this repository's CUDA path, headline workload
    python bench.py --workload {small_lattice,rbm,potts,potts_program,lattice} ...   # the other configurations
    python bench.py --impl reference [--workload ...] --steps K ...    # the CPU restatement of the reference's path (oracle/)

Headline workload (`sparse_ising`): sparse random 8-regular Ising graph, 2^20 spins, ~4.19 M edges, greedy-coloured
blocks, 4096 chains per GPU, first and second moments every sweep.  One step = one Gibbs sweep over every block for
every chain, followed by the moment observer.  `value` is site updates per second with the chain state resident in
HBM; `e2e` is the same metric through the host-buffer calls (initial state uploaded from pinned host memory, moment
sums read back).  Every CUDA line carries `roofline`, `cpu_baseline` (N = 1) and `e2e`; `parity_check` reports the
oracle following a slice of the chains of the very state that was benchmarked.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_NODES = 1 << 20
DEGREE = 8
CHAINS_PER_GPU = 4096
SEED = 0x5EED0002
METRIC = "gibbs_site_updates_per_sec"
UNIT = "site-updates/s"
# DRAM bytes per site update of k_spin_lut: dram__bytes_read.sum + dram__bytes_write.sum of one launch under ncu on the
# 2^18-spin, 4096-chain, 8-regular case (profiles/k_spin_lut_sparse_ising.md), divided by that launch's site updates.
# A random graph has no cross-node reuse, so the traffic of a launch grows in proportion to its site updates.
LUT_DRAM_BYTES_PER_UPDATE = 8.92
# The same for one k_lattice_update_sliced launch on a 16384^2 lattice, 16 chains (profiles/k_lattice_update_sliced_ising_bitpacked.md)
# and one k_potts_update launch on a 64^3 lattice, 1024 chains (profiles/k_potts_update_potts128.md); both kernels stream
# their state once per launch, so the traffic of a launch grows in proportion to its site updates.
LATTICE_DRAM_BYTES_PER_UPDATE = 0.2375
POTTS_DRAM_BYTES_PER_UPDATE = 2.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default: 500 sweeps for sparse_ising, a workload-specific count otherwise)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--nodes", type=int, default=N_NODES, help="graph size (default: the benchmark configuration)")
    ap.add_argument("--chains", type=int, default=None, help="chains per GPU (default: the configuration's)")
    ap.add_argument("--state-format", default="int8", choices=["int8", "bitpacked"],
                    help="sparse_ising: int8 (default) = one byte per spin and chain, the HBM-bound format the roofline target is quoted on; "
                         "bitpacked = sweeps on the bit-packed mirror (THRML_OPT_STATE_FORMAT), more site updates per second, bound by instruction issue")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle's check of a chain slice of the benchmarked state")
    ap.add_argument("--workload", default="sparse_ising", choices=["sparse_ising", "rbm", "lattice", "potts", "potts_program", "small_lattice", "mixed"],
                    help="sparse_ising = the headline configuration; rbm = dense bipartite CD-1 on the tensor cores; lattice = one bit-packed 2-D Ising "
                         "lattice sharded by row stripes with halo exchange; potts = implicit 3-D Potts lattice; small_lattice = 32 x 32 torus, 256 chains")
    ap.add_argument("--side", type=int, default=None, help="lattice side (lattice / potts / potts_program workloads)")
    ap.add_argument("--graph", default="regular", choices=["regular", "random"],
                    help="sparse_ising workload: degree-regular graph (the headline) or a random graph with that mean degree")
    ap.add_argument("--degree", type=int, default=DEGREE, help="stubs per node of the sparse graph (the headline uses 8; above 8 the "
                    "blocks leave the threshold-table kernel for the sequential-sum kernel)")
    ap.add_argument("--dense-tiles", default="auto", choices=["auto", "pair", "single"],
                    help="rbm workload: CTA pairs sharing 256-row tiles (tcgen05 cta_group::2), one CTA per 128-row tile, or chosen per launch")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = {"sparse_ising": 500, "rbm": 200, "lattice": 50, "potts": 20, "potts_program": 20, "small_lattice": 20, "mixed": 20}[args.workload]
    if args.chains is None:
        args.chains = {"sparse_ising": CHAINS_PER_GPU, "rbm": 8192, "lattice": 16, "potts": 1024, "potts_program": 1024, "small_lattice": 256, "mixed": 4096}[args.workload]
    if args.side is None:
        args.side = {"lattice": 32768, "potts": 128, "potts_program": 32, "mixed": 512}.get(args.workload, 0)
    return args


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 200 ms while the timed region runs."""
    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, device):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(device), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        rows = [r for t, r in self.rows if t0 <= t <= t1 + 0.3] or [r for _, r in self.rows]
        sm, mx, reasons = [], [], set()
        for r in rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return json.load(open(path)), True
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, False


def hbm_peak():
    peaks, measured = measured_peaks()
    return float(peaks["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)" if measured else "fallback (6.65 TB/s; MEASURED_PEAKS.json absent)"


def hbm_roofline(updates_per_launch, bytes_per_update, launch_ms, kernel, note=None, dram_bytes_per_update=None, dram_provenance=None):
    """`achieved` = algorithmic bytes of one launch / its CUDA-event duration; `traffic` = DRAM bytes of one launch from
    an ncu capture scaled by site updates (null when no capture matches this kernel and shape)."""
    peak, src = hbm_peak()
    algo = updates_per_launch * bytes_per_update
    achieved = algo / (launch_ms * 1e-3) / 1e9
    out = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_source": src, "kernel": kernel,
           "algorithmic_bytes_per_launch": algo, "bytes_per_update": bytes_per_update, "launch_ms": launch_ms}
    if dram_bytes_per_update is not None:
        out["traffic"] = dram_bytes_per_update * updates_per_launch
        out["dram_frac"] = out["traffic"] / (launch_ms * 1e-3) / 1e9 / peak
        out["traffic_provenance"] = dram_provenance
    if note:
        out["note"] = note
    return out


def pinned(torch, array):
    t = torch.empty(array.shape, dtype=getattr(torch, str(array.dtype)), pin_memory=True)
    t.numpy()[...] = array
    return t


def pinned_u32(torch, array):
    """uint32 numpy data in pinned host memory (held as int32 storage; the bytes are what matters)."""
    t = torch.empty(array.shape, dtype=torch.int32, pin_memory=True)
    t.numpy().view(np.uint32)[...] = array
    return t


# -----------------------------------------------------------------------------------------------------------
# CPU legs: the oracle (a C++ restatement of the reference's per-block op sequence: f32 0/1 state, materialised
# gathers, per-sample moment loop) on this box's host cores.  Each `cpu_*` function builds the workload in the oracle
# and returns step(i) -> site updates done; cpu_sample times a bounded number of steps.
# -----------------------------------------------------------------------------------------------------------
def cpu_sparse(args, threads, model=None):
    from oracle import oracle as O
    from thrml_rs_b200 import workloads as W
    if model is None:
        model = W.sparse_ising(args.nodes, args.degree, SEED, regular=args.graph == "regular")
    om = W.fill_ising(O.Model(np.zeros(model["n"], np.int32)), model)
    st = O.State(om, threads, 0, threads=threads)
    st.randomize(1)
    mom = O.Moments.from_arrays(om, *W.ising_moment_arrays(model))

    def step(i):
        st.run_blocks(200 + i, 1)
        mom.observe(st)
        return model["n"] * threads

    return step, f"one step = one sweep + moment observation of {threads} chains (one per host thread) on the full {model['n']}-spin graph", om


def cpu_small_lattice(args, threads):
    from oracle import oracle as O
    import __graft_entry__ as graft
    T = graft.load_package()
    m = small_lattice_model(T)
    om = O.Model(np.zeros(m["n"], np.int32))
    for blk in m["blocks"]:
        om.add_free_block(blk)
    om.add_ising(np.arange(m["n"]), m["b"], m["edges"], m["J"], 1.0)
    om.compile()
    chains = args.chains
    st = O.State(om, chains, 0, threads=threads)
    mom = O.Moments.from_arrays(om, *m["spec"])

    def step(i):
        st.hinton_init([0, 1], m["biases"], 1.0, 7 + i)
        st.sample_with_observation(2026 + i, 200, 801, 1, moments=mom)
        return m["n"] * chains * 1000

    return step, f"one step = the whole configuration: hinton_init + schedule (200, 801, 1) with moments, {chains} chains over {threads} threads", om


def cpu_rbm(args, threads):
    from oracle import oracle as O
    from thrml_rs_b200 import workloads as W
    model = W.rbm_ising()
    om = W.fill_ising(O.Model(np.zeros(model["n"], np.int32)), model)
    chains = 2 * threads
    st = O.State(om, chains, 0, threads=threads)
    rng = np.random.default_rng(3)
    v0 = (rng.random((chains, model["n_visible"])) < 0.13).astype(np.float32)
    s = lambda x: 2.0 * x - 1.0

    def step(i):
        k0, k1 = [int(k) for k in O.rng_split(500 + i, 2)]
        st.set_block(0, v0)
        st.sample_single_block(1, k0)
        pos = s(v0).T @ s(st.get_block(1)) / chains
        st.sample_blocks(k1)
        neg = s(st.get_block(0)).T @ s(st.get_block(1)) / chains
        return chains * (2 * model["n_hidden"] + model["n_visible"]) + 0 * float(pos[0, 0] + neg[0, 0])

    return step, f"one step = CD-1 (h0 | v0, one sweep, both correlation matrices with a BLAS f32 product) on {chains} chains over {threads} threads", om


def potts_arrays(side, K, seed=0x5EED0004):
    rng = np.random.default_rng(seed)
    tables = rng.normal(0, 0.3, (3, K, K)).astype(np.float32)
    unary = rng.normal(0, 0.1, (side ** 3, K)).astype(np.float32)
    return tables, unary


def potts_explicit(builder_cls, side, K, tables, unary):
    """The factor program the reference would build: unary CategoricalEBMFactor + one [n, K, K] pair factor per direction."""
    n = side ** 3
    idx = np.arange(n).reshape(side, side, side)
    colour = (np.add.outer(np.add.outer(np.arange(side), np.arange(side)), np.arange(side)) % 2).ravel()
    bld = builder_cls(np.full(n, K, np.int32))
    for c in (0, 1):
        bld.add_free_block(np.flatnonzero(colour == c))
    bld.add_discrete_factor([], [np.arange(n)], unary.reshape(n, K, 1))
    for d in range(3):
        bld.add_discrete_factor([], [idx.ravel(), np.roll(idx, -1, axis=d).ravel()], np.broadcast_to(tables[d], (n, K, K)).copy())
    bld.compile()
    return bld


def cpu_potts(args, threads):
    from oracle import oracle as O
    side = min(args.side, 48)  # the explicit program materialises [n, 6, K*K] weights per block: 128^3 would need 5 GB
    K = 10
    tables, unary = potts_arrays(side, K)
    om = potts_explicit(O.Model, side, K, tables, unary)
    st = O.State(om, threads, 0, threads=threads)
    st.randomize(5)

    def step(i):
        st.run_blocks(300 + i, 1)
        return side ** 3 * threads

    return step, f"one step = one sweep of {threads} chains (one per host thread) of the explicit factor program on a {side}^3 lattice (per-update cost does not depend on the side)", om


def cpu_lattice(args, threads):
    from oracle import oracle as O
    import __graft_entry__ as graft
    T = graft.load_package()
    side = min(args.side, 1024)  # the explicit program holds per-node tables: 32768^2 cannot be built
    n = side * side
    _, edges, colour = T.lattice_edges(side, True)
    om = O.Model(np.zeros(n, np.int32))
    for c in (0, 1):
        om.add_free_block(np.flatnonzero(colour == c))
    om.add_ising(np.arange(n), np.zeros(n, np.float32), edges, np.full(len(edges), 0.4407, np.float32), 1.0)
    om.compile()
    chains = max(threads, 16) // 16 * 16
    st = O.State(om, chains, 0, threads=threads)
    st.randomize(11)

    def step(i):
        st.run_blocks(50 + i, 1)
        return n * chains

    return step, f"one step = one sweep of {chains} chains over {threads} threads of the explicit Ising program on a {side}^2 torus (per-update cost does not depend on the side)", om


def cpu_mixed(args, threads):
    from oracle import oracle as O
    from thrml_rs_b200 import workloads as W
    side = min(args.side, 256)
    model = W.spin_category_checkerboard(side, 4)
    om = W.fill_factors(O.Model(model["kinds"], model["dtype_order"]), model)
    st = O.State(om, threads, 0, threads=threads)
    st.randomize(5)

    def step(i):
        st.run_blocks(300 + i, 1)
        return model["n"] * threads

    return step, f"one step = one sweep of {threads} chains (one per host thread) of the same factor program on a {side}^2 grid (per-update cost does not depend on the side)", om


CPU_LEGS = {"mixed": cpu_mixed, "sparse_ising": cpu_sparse, "small_lattice": cpu_small_lattice, "rbm": cpu_rbm, "potts": cpu_potts, "potts_program": cpu_potts, "lattice": cpu_lattice}


def cpu_sample(step, target_seconds, max_steps, warmup=1):
    for i in range(warmup):
        step(-1 - i)
    done, updates, t0 = 0, 0.0, time.time()
    while done < max_steps:
        updates += step(done)
        done += 1
        if time.time() - t0 > target_seconds:
            break
    dt = time.time() - t0
    return updates / dt, done, dt


def cpu_baseline(args, threads, target_seconds=12.0, **kw):
    step, what, om = CPU_LEGS[args.workload](args, threads, **kw)
    value, done, dt = cpu_sample(step, target_seconds, 200)
    return {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"{what}; {done} steps, {dt:.1f} s"}, om


def run_reference(args):
    """The CPU restatement of the reference's path on all host cores, W warm-up and K timed steps of a bounded sample of
    the workload (one step is described in `cpu_baseline.sample`); K is cut when the run would pass about two minutes."""
    threads = os.cpu_count() or 1
    step, what, _ = CPU_LEGS[args.workload](args, threads)
    for i in range(max(args.warmup, 0)):
        step(-1 - i)
    t0 = time.time()
    first = step(0)
    t_first = time.time() - t0
    steps = max(1, min(args.steps, int(120.0 / max(t_first, 1e-3))))
    updates = first
    for i in range(1, steps):
        updates += step(i)
    dt = time.time() - t0
    value = updates / dt
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": max(args.warmup, 0),
            "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "strong" if args.workload == "lattice" else "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": workload_config(args), "config_timed": what,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": f"{what}; {steps} steps timed, {dt:.1f} s"},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if steps != args.steps:
        line["steps_requested"] = args.steps
    return line


def workload_config(args, model=None, world=None):
    world = world or args.gpus
    if args.workload == "sparse_ising":
        kind = f"{args.degree}-regular" if args.graph == "regular" else f"random, mean degree {args.degree}"
        cfg = {"workload": f"sparse random {kind} Ising graph, greedy-coloured blocks, <s_i> and <s_i s_j> accumulated every sweep",
               "nodes": int(args.nodes), "chains_per_gpu": int(args.chains), "global_chains": int(args.chains * world),
               "state_format": "int8 (one byte per spin and chain, chains innermost)",
               "parallelism": f"chains sharded over {world} GPU(s), one allreduce of the moment sums", "l2": "inputs larger than L2 (state is nodes x chains bytes)"}
        if model is not None:
            cfg["edges"] = int(len(model["edges"]))
            cfg["blocks"] = len(model["blocks"])
        return cfg
    if args.workload == "small_lattice":
        return {"workload": "32 x 32 periodic Ising lattice, 256 chains, hinton_init + 1000 sweeps (200 warm-up, 801 samples) with moments per step",
                "chains": int(args.chains), "l2": "cache-resident (256 KiB of state): L2 is not flushed, the configuration itself is cache-resident"}
    if args.workload == "rbm":
        return {"workload": "bipartite RBM-style Ising EBM, CD-1 per step", "visible": 784, "hidden": 4096, "chains_per_gpu": int(args.chains), "global_chains": int(args.chains * world),
                "parallelism": f"chains sharded over {world} GPU(s), one allreduce of the two correlation matrices per step",
                "l2": "operands (6.4 MB couplings, 13-67 MB states) fit in L2: a tensor-pipe measurement, not an HBM one"}
    if args.workload == "mixed":
        return {"workload": "spin / 4-state checkerboard with three-spin terms (not a BASELINE configuration: the general spin and the warp-per-node categorical kernels)",
                "side": int(args.side), "categories": 4, "chains": int(args.chains), "l2": "state (1 GiB at side 512, 4096 chains) larger than L2"}
    if args.workload in ("potts", "potts_program"):
        return {"workload": "3-D periodic Potts-like lattice, K = 10, shared direction tables" + (", as an explicit factor program" if args.workload == "potts_program" else ", category marginals every sweep"),
                "side": int(args.side), "categories": 10, "chains_per_gpu": int(args.chains), "global_chains": int(args.chains * world),
                "parallelism": f"chains sharded over {world} GPU(s), one allreduce of the category counts", "l2": "state (2 GiB at side 128) larger than L2" if args.side >= 64 else "cache-resident"}
    return {"workload": "2-D periodic Ising lattice, bit-packed, checkerboard blocks, row stripes with halo exchange, magnetisation and energy recorded every sweep",
            "side": int(args.side), "chains": int(args.chains), "stripe_rows": int(args.side // world), "parallelism": f"rows sharded over {world} GPU(s), halo rows by NCCL point-to-point",
            "halo_bytes_per_half_sweep_per_neighbour": int(args.side // 2 // 8 * args.chains), "l2": "state (2 GiB at side 32768) larger than L2"}


def base_line(args, value, ms_per_step, world, dtype, scaling="weak"):
    return {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic"}


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    import __graft_entry__ as graft

    if args.impl == "reference":
        if rank != 0:
            return
        graft.load_package()
        print(json.dumps(run_reference(args)), flush=True)
        return

    import torch
    T = graft.load_package()
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = T.default_context(local_rank)
    comm = T.Comm.from_torch(dist, ctx) if dist else None
    env = dict(T=T, torch=torch, args=args, rank=rank, world=world, device=local_rank, dist=dist, ctx=ctx, comm=comm)
    if args.workload in ("small_lattice", "potts_program", "mixed") and world > 1:
        # these configurations are replicas: every rank would run the same independent problem
        if rank == 0:
            print(json.dumps({"metric": METRIC, "unavailable": f"--workload {args.workload} runs on one GPU (replicas only); use --gpus 1"}), flush=True)
    else:
        out = {"sparse_ising": run_sparse, "rbm": run_rbm, "small_lattice": run_small_lattice, "potts_program": run_potts_program, "potts": run_potts,
               "lattice": run_lattice, "mixed": run_mixed}[args.workload](**env)
        if rank == 0:
            print(json.dumps(out), flush=True)
    if comm is not None:
        comm.close()
    if dist:
        dist.barrier()
        dist.destroy_process_group()


def timed(torch, stream, fn, sync):
    """fn() between two CUDA events on `stream`, with a synchronisation on both sides; returns milliseconds."""
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    ev0.record(stream)
    fn()
    ev1.record(stream)
    sync()
    return ev0.elapsed_time(ev1)


def max_over_ranks(torch, dist, x):
    if not dist:
        return x
    t = torch.tensor([x], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


# -----------------------------------------------------------------------------------------------------------
# Headline: sparse Ising, chains sharded over the GPUs.
# -----------------------------------------------------------------------------------------------------------
def run_sparse(T, torch, args, rank, world, device, dist, ctx, comm):
    from thrml_rs_b200 import workloads as W
    # the two steps before the path (greedy colouring, slot tables) run on the device; the parity check below follows the
    # oracle's own host compilation of the same blocks, so it covers these tables at full size
    t0 = time.perf_counter()
    model = W.sparse_ising(args.nodes, args.degree, SEED, regular=args.graph == "regular", ctx=ctx)
    t1 = time.perf_counter()
    n, chains = model["n"], args.chains
    builder = W.fill_ising(T.Builder(np.zeros(n, np.int32)), model, ctx=ctx)
    prepare = {"where": "device", "graph_and_colouring_s": round(t1 - t0, 3), "add_factors_and_compile_s": round(time.perf_counter() - t1, 3)}
    program = T.Program(builder, ctx)
    if args.state_format == "bitpacked":
        program.set_option(T.OPT_STATE_FORMAT, 1)
    n_blocks = len(model["blocks"])
    state = T.ChainState(program, chains, chain_offset=rank * chains)
    moments = T.Moments.from_arrays(program, *W.ising_moment_arrays(model))
    biases = np.concatenate([model["b"][blk] for blk in model["blocks"]])
    state.hinton_init(list(range(n_blocks)), biases, model["beta"], SEED)
    stream = torch.cuda.ExternalStream(ctx.stream)

    def step(i):
        state.sample_with_observation(1000 + i, 1, 1, 1, moments=moments)  # one sweep, then observe

    def barrier():
        ctx.synchronize()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()

    for i in range(max(args.warmup, 3)):
        step(i)
    if comm:
        moments.allreduce(comm)  # same size and type as the timed one: connections and buffers are set up here
    barrier()
    moments.reset()
    sampler = ClockSampler(device) if rank == 0 else None
    ev0, ev1, eva = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    barrier()
    t_wall0 = time.time()
    ev0.record(stream)
    for i in range(args.steps):
        step(100 + i)
    eva.record(stream)
    if comm:  # the single allreduce of the moment sums, on the engine's stream after the sweeps
        moments.allreduce(comm)
    ev1.record(stream)
    barrier()
    t_wall1 = time.time()
    ms = max_over_ranks(torch, dist, ev0.elapsed_time(ev1))
    allreduce_ms = max_over_ranks(torch, dist, eva.elapsed_time(ev1)) if comm else 0.0
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    # dominant kernel alone: sweeps without the observer, timed with events on the launching stream
    sweep_iters = max(5, min(args.steps, 20))
    sweep_ms = timed(torch, stream, lambda: state.run_blocks(7, sweep_iters), barrier) / sweep_iters

    updates_per_step = float(n) * chains
    result = base_line(args, updates_per_step * world * args.steps / (ms * 1e-3), ms / args.steps, world, "u8")
    other_rows = moments.fused_info()[1]
    result.update({"config": workload_config(args, model, world), "clocks": clocks, "allreduce_ms": allreduce_ms, "prepare": prepare,
                   "gpu_launches": args.steps * (n_blocks + (1 if other_rows > 0 else 0)) + (3 if comm else 0)})
    # roofline of the block-update kernel.  Algorithmic bytes per site update: one byte per neighbour read and one written,
    # plus the per-node parameters (4 B index + 4 B coupling per slot, bias) and observer rows amortised over the chains.
    kinds = [program.block_kernel(b) for b in range(n_blocks)]
    mean_deg = 2.0 * len(model["edges"]) / n
    bytes_per_update = (mean_deg + 1.0) + 10.0 * mean_deg / chains
    packed = args.state_format == "bitpacked" and all(k == 1 for k in kinds) and chains > 1008
    if packed:  # one bit per neighbour read and one written; the same parameters
        bytes_per_update = (mean_deg + 1.0) / 8.0 + 10.0 * mean_deg / chains
    result["config"]["state_format"] = "bit-packed mirror (THRML_OPT_STATE_FORMAT = 1)" if packed else "int8"
    kernel = "k_packed_lut" if packed else "k_spin_lut" if all(k == 1 for k in kinds) else ("k_spin_seq" if all(k == 4 for k in kinds) else ("k_spin_hybrid" if all(k in (1, 4, 6) for k in kinds) else "k_spin_generic"))
    if packed:
        result["dtype"] = "1-bit spins, u32 thresholds"
    profiled = kernel == "k_spin_lut" and args.degree == DEGREE and args.graph == "regular" and chains == CHAINS_PER_GPU
    # The launches of the timed region are the update kernel with the moment observer fused in (the 80/chains term of the
    # traffic model is its rows and parameters): their average duration is the step time over the launches of a step, minus
    # the one allreduce when there is one.  `update_only` is the same kernel without the observer, timed on its own.
    step_launches = n_blocks + (1 if other_rows > 0 else 0)
    fused_launch_ms = (ms - allreduce_ms) / args.steps / step_launches
    provenance = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one k_spin_lut launch on the 2^18-spin, 4096-chain, 8-regular case "
                  "(profiles/k_spin_lut_sparse_ising.md), scaled by site updates") if profiled else None
    result["roofline"] = hbm_roofline(updates_per_step / n_blocks, bytes_per_update, fused_launch_ms, kernel + " (moment observer fused in)",
                                      dram_bytes_per_update=LUT_DRAM_BYTES_PER_UPDATE if profiled else None, dram_provenance=provenance)
    only = hbm_roofline(updates_per_step / n_blocks, bytes_per_update, sweep_ms / n_blocks, kernel,
                        dram_bytes_per_update=LUT_DRAM_BYTES_PER_UPDATE if profiled else None, dram_provenance=provenance)
    result["roofline"].update({"launches_per_sweep": n_blocks, "sweep_ms": sweep_ms,
                               "update_only": {k: only[k] for k in ("achieved", "frac", "launch_ms", "kernel") if k in only} | ({"dram_frac": only["dram_frac"]} if "dram_frac" in only else {})})

    if not args.no_e2e:
        del state, moments
        result.update(sparse_end_to_end(T, torch, program, model, chains, rank, ctx, args, dist, comm))
        state = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"], om = cpu_baseline(args, os.cpu_count() or 1, model=model)
        if not args.no_parity:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import fullsize_checks as F
            from oracle import oracle as O
            state = T.ChainState(program, chains, chain_offset=rank * chains)
            result["parity_check"] = F.sparse_ising_check(T, O, model, program, state, chains, oracle_model=om, threads=os.cpu_count() or 1)
    return result


def sparse_end_to_end(T, torch, program, model, chains, rank, ctx, args, dist, comm):
    """estimate-moments through the host-buffer calls: upload the initial chain state of every block from pinned host
    memory, `steps` sweeps with the moment observer, (allreduce,) read the sums back.  Primary figure: the state travels
    bit-packed (thrml_state_upload_packed); also reported: one byte per spin (thrml_state_upload_u8_many) and the
    reference's own flow, hinton_init from the host's bias vector (ising.rs:602-673) followed by estimate_moments."""
    from thrml_rs_b200 import workloads as W
    n_blocks = len(model["blocks"])
    rng = np.random.default_rng(1 + rank)
    words = (chains + 31) // 32
    # independent random start states per variant, generated directly in each variant's host layout
    host_u8 = [pinned(torch, rng.integers(0, 2, (chains, len(blk)), dtype=np.uint8)) for blk in model["blocks"]]
    host_bits = [pinned_u32(torch, rng.integers(0, 1 << 32, (len(blk), words), dtype=np.uint32)) for blk in model["blocks"]]
    biases = np.concatenate([model["b"][blk] for blk in model["blocks"]])
    steps = args.steps
    world = dist.get_world_size() if dist else 1
    d2h = (model["n"] + len(model["edges"])) * 8
    blocks = list(range(n_blocks))
    spec = W.ising_moment_arrays(model)
    sums_host = [torch.empty(int(k), dtype=torch.int64, pin_memory=True) for k in spec[0]]

    def run(upload):
        best = None
        for rep in range(2):
            state = T.ChainState(program, chains, chain_offset=rank * chains)
            moments = T.Moments.from_arrays(program, *spec)
            ctx.synchronize()
            if dist:
                dist.barrier()
            t0 = time.perf_counter()
            upload(state)
            state.sample_with_observation(5, 1, steps, 1, moments=moments)  # `steps` x (sweep, observe)
            if comm:
                moments.allreduce(comm)
            for t, buf in enumerate(sums_host):
                moments.read(t, buf.numpy())
            ctx.synchronize()
            dt = max_over_ranks(torch, dist, time.perf_counter() - t0)
            best = dt if best is None else min(best, dt)
            del state, moments
        return best

    updates = float(model["n"]) * chains * world * steps
    t_bits = run(lambda st: st.upload_packed(blocks, [t.numpy().view(np.uint32) for t in host_bits]))
    t_u8 = run(lambda st: st.upload_many(blocks, [t.numpy() for t in host_u8]))
    t_hint = run(lambda st: st.hinton_init(blocks, biases, model["beta"], 77))
    h2d_bits = sum(int(t.numel()) * 4 for t in host_bits)
    e2e = {"value": updates / t_bits, "unit": UNIT, "h2d_bytes_per_step": h2d_bits / steps, "d2h_bytes_per_step": d2h / steps, "seconds": t_bits,
           "call": "thrml_state_upload_packed (pinned host bits -> device) + thrml_sample_with_observation(moments) + (thrml_moments_allreduce) + thrml_moments_read"}
    variants = {"u8_upload": {"value": updates / t_u8, "h2d_bytes_per_step": sum(int(t.numel()) for t in host_u8) / steps, "seconds": t_u8,
                              "call": "thrml_state_upload_u8_many instead of the packed upload"},
                "hinton_init": {"value": updates / t_hint, "h2d_bytes_per_step": biases.nbytes / steps, "seconds": t_hint,
                                "call": "thrml_hinton_init from the host's bias vector instead of an upload (the reference's estimate_moments flow)"}}
    return {"e2e": e2e, "e2e_variants": variants}


# -----------------------------------------------------------------------------------------------------------
# Dense bipartite (RBM) configuration.
# -----------------------------------------------------------------------------------------------------------
def run_rbm(T, torch, args, rank, world, device, dist, ctx, comm):
    """784 visible x 4096 hidden spins, bf16 couplings, 8192 chains, CD-1 per step (h0 | v0, one Gibbs sweep, positive and
    negative correlations).  Reported against the measured bf16 GEMM peak."""
    from thrml_rs_b200 import workloads as W
    model = W.rbm_ising()
    nv, nh, chains = model["n_visible"], model["n_hidden"], args.chains
    builder = W.fill_ising(T.Builder(np.zeros(model["n"], np.int32)), model)
    program = T.Program(builder, ctx)
    assert program.enable_dense(False) == 2
    program.set_option(T.OPT_DENSE_TILES, {"single": 0, "pair": 1, "auto": 2}[args.dense_tiles])
    # with several GPUs every rank holds `chains` chains of its own data (global chain ids rank * chains + c) and every step ends
    # with one allreduce of the two correlation matrices (thrml_cd1_step_comm): weak scaling
    rng = np.random.default_rng(3 + rank)
    v0 = (rng.random((chains, nv)) < 0.13).astype(np.uint8)
    data, state = T.ChainState(program, chains, rank * chains), T.ChainState(program, chains, rank * chains)
    data.upload(0, v0)
    stream = torch.cuda.ExternalStream(ctx.stream)

    def step(i):
        state.cd1_step(0, 1, None, 500 + i, want_stats=False, data=data, comm=comm)  # v0 is read from the resident data state

    def sync():
        ctx.synchronize()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()

    for i in range(max(args.warmup, 3)):
        step(i)
    sampler = ClockSampler(device) if rank == 0 else None
    t0 = time.time()
    ms = max_over_ranks(torch, dist, timed(torch, stream, lambda: [step(100 + i) for i in range(args.steps)], sync)) / args.steps
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if sampler else None
    flop = 5 * 2.0 * chains * nv * nh  # 3 field GEMMs + 2 correlation GEMMs, per GPU
    updates = chains * (nh + nv + nh) * world
    if world > 1:
        peaks, measured = measured_peaks()
        peak = float(peaks["bf16_tflops"])
        achieved = flop / (ms * 1e-3) / 1e12
        out = base_line(args, updates / (ms * 1e-3), ms, world, "bf16 couplings x +-1 states, f32 accumulate; u8 x u8 -> s32 correlations")
        out.update({"config": workload_config(args, world=world), "clocks": clocks, "gpu_launches": args.steps * 10,  # + allreduce and scale
                    "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                                 "peak_source": "measured burst bf16 GEMM (MEASURED_PEAKS.json)" if measured else "fallback 1590 (MEASURED_PEAKS.json absent)",
                                 "flop_per_step": flop, "note": "per GPU; the step includes one ncclAllReduce of 2 x 784 x 4096 f32"}})
        return out
    peaks, measured = measured_peaks()
    peak = float(peaks["bf16_tflops"])
    achieved = flop / (ms * 1e-3) / 1e12
    # end to end: upload v0 from pinned host memory, CD-1, read both correlation matrices back
    hv = pinned(torch, v0)
    corr_host = (torch.empty((nv, nh), dtype=torch.float32, pin_memory=True), torch.empty((nv, nh), dtype=torch.float32, pin_memory=True))
    best = None
    for rep in range(3):
        ctx.synchronize()
        ta = time.perf_counter()
        state.cd1_step(0, 1, hv.numpy(), 900 + rep, out=(corr_host[0].numpy(), corr_host[1].numpy()))
        dt = time.perf_counter() - ta
        best = dt if best is None else min(best, dt)
    out = base_line(args, updates / (ms * 1e-3), ms, 1, "bf16 couplings x +-1 states, f32 accumulate; u8 x u8 -> s32 correlations")
    out.update({"config": workload_config(args), "clocks": clocks, "gpu_launches": args.steps * 8,  # three field GEMMs, two correlation GEMMs, three clears of the one counts
                "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                             "peak_source": "measured burst bf16 GEMM (MEASURED_PEAKS.json)" if measured else "fallback 1590 (MEASURED_PEAKS.json absent)",
                             "flop_per_step": flop, "note": "3 bf16 field GEMMs + 2 int8 correlation GEMMs counted at 2*M*N*K each"},
                "e2e": {"value": updates / best, "unit": UNIT, "h2d_bytes_per_step": chains * nv, "d2h_bytes_per_step": 2 * nv * nh * 4, "seconds": best,
                        "call": "thrml_cd1_step with the visible data in pinned host memory and both correlation matrices read back"}})
    if not args.no_cpu_baseline:
        out["cpu_baseline"], _ = cpu_baseline(args, os.cpu_count() or 1)
    if not args.no_parity:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import fullsize_checks as F
        from oracle import oracle as O
        del state, data
        out["parity_check"] = F.dense_check(T, O, n_visible=nv, n_hidden=nh, chains=1024, tiles={"single": 0, "pair": 1, "auto": 2}[args.dense_tiles], ctx=ctx)
    return out


# -----------------------------------------------------------------------------------------------------------
# 32 x 32 torus, 256 chains (the configuration the reference itself could run on a CPU).
# -----------------------------------------------------------------------------------------------------------
def small_lattice_model(T):
    rng = np.random.default_rng(0x5EED0001)
    side, edges, colour = T.lattice_edges(32, True)
    n = side * side
    b = rng.normal(0, 0.1, n).astype(np.float32)
    J = np.full(len(edges), 0.44, np.float32)
    blocks = [np.flatnonzero(colour == c) for c in (0, 1)]
    rows_per_type = np.array([n, len(edges)], dtype=np.int64)
    row_ptr = np.concatenate([np.arange(n + 1), n + 2 * np.arange(1, len(edges) + 1)]).astype(np.int64)
    members = np.concatenate([np.arange(n), edges.ravel()]).astype(np.int64)
    return dict(n=n, edges=edges, b=b, J=J, blocks=blocks, spec=(rows_per_type, row_ptr, members), biases=np.concatenate([b[blk] for blk in blocks]))


def run_small_lattice(T, torch, args, rank, world, device, dist, ctx, comm):
    """32 x 32 periodic Ising lattice (J = 0.44, biases N(0, 0.1^2), beta = 1), 256 chains, hinton_init, schedule
    (200 warm-up, 801 samples, 1 step) = 1000 sweeps with <s_i> and <s_i s_j> observed: the whole problem is cache-resident,
    so this measures launch and barrier latency, not bandwidth.  One timed step = the whole 1000-sweep schedule."""
    m = small_lattice_model(T)
    n, chains = m["n"], args.chains
    bld = T.Builder(np.zeros(n, np.int32))
    for blk in m["blocks"]:
        bld.add_free_block(blk)
    bld.add_ising(np.arange(n), m["b"], m["edges"], m["J"], 1.0)
    bld.compile()
    program = T.Program(bld, ctx)
    state = T.ChainState(program, chains)
    moments = T.Moments.from_arrays(program, *m["spec"])
    stream = torch.cuda.ExternalStream(ctx.stream)

    def step(i):
        state.hinton_init([0, 1], m["biases"], 1.0, 7 + i)
        state.sample_with_observation(2026 + i, 200, 801, 1, moments=moments)

    def sync():
        ctx.synchronize()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    reps = max(1, args.steps)
    launches0 = state.launch_counts()
    sampler = ClockSampler(device)
    t0 = time.time()
    ms = timed(torch, stream, lambda: [step(10 + i) for i in range(reps)], sync) / reps
    t1 = time.time()
    clocks = sampler.stop(t0, t1)
    launches1 = state.launch_counts()
    updates = float(n) * chains * 1000
    # end to end: the same step as the host sees it — biases in, moment sums out, wall clock
    best = None
    for rep in range(3):
        moments.reset()
        sync()
        ta = time.perf_counter()
        step(50 + rep)
        moments.read(0)
        moments.read(1)
        dt = time.perf_counter() - ta
        best = dt if best is None else min(best, dt)
    out = base_line(args, updates / (ms * 1e-3), ms, 1, "u8")
    out.update({"config": workload_config(args), "clocks": clocks,
                # one k_hinton per block and step, plus the update launches the state counted (per-block and persistent)
                "gpu_launches": reps * 2 + sum(launches1) - sum(launches0),
                "roofline": hbm_roofline(updates, 5.0 + 48.0 / chains, ms, "k_spin_lut_sliced",
                                         note="nominal: the state lives in shared memory for the whole schedule, HBM sees 256 KiB in and out per launch; bound by instruction latency between CTA barriers"),
                "e2e": {"value": updates / best, "unit": UNIT, "h2d_bytes_per_step": int(m["biases"].nbytes), "d2h_bytes_per_step": int((n + len(m["edges"])) * 8), "seconds": best,
                        "call": "thrml_hinton_init (host biases) + thrml_sample_with_observation(moments) + thrml_moments_read"}})
    if not args.no_cpu_baseline:
        out["cpu_baseline"], _ = cpu_baseline(args, os.cpu_count() or 1, target_seconds=25.0)
    return out


# -----------------------------------------------------------------------------------------------------------
# Potts: explicit factor program (general categorical kernels) and implicit lattice.
# -----------------------------------------------------------------------------------------------------------
def run_potts_program(T, torch, args, rank, world, device, dist, ctx, comm):
    """The same kind of model as `potts`, but as the explicit factor program the reference would build
    (FactorSamplingProgram over a unary CategoricalEBMFactor and one [n, K, K] pair factor per direction, crates/thrml-models/src/
    factor.rs:153-184), at 32^3 nodes (the per-edge weight tensors are 39 MB there; 2.5 GB per block at 128^3): the general
    categorical kernels instead of the implicit lattice."""
    side, K, chains = args.side, 10, args.chains
    n = side ** 3
    tables, unary = potts_arrays(side, K)
    program = T.Program(potts_explicit(T.Builder, side, K, tables, unary), ctx)
    kinds = [program.block_kernel(b) for b in range(2)]
    state = T.ChainState(program, chains)
    state.randomize(5)
    stream = torch.cuda.ExternalStream(ctx.stream)

    def sync():
        ctx.synchronize()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        state.sample_blocks(i)
    ms = timed(torch, stream, lambda: [state.sample_blocks(100 + i) for i in range(args.steps)], sync) / args.steps
    updates = float(n) * chains
    # end to end: categories in (pinned host bytes), `steps` sweeps, categories out
    rng = np.random.default_rng(9)
    host = [pinned(torch, rng.integers(0, K, (chains, n // 2), dtype=np.uint8)) for _ in range(2)]
    sync()
    ta = time.perf_counter()
    state.upload_many([0, 1], [h.numpy() for h in host])
    state.run_blocks(55, args.steps)
    back = [state.download(b, np.uint8) for b in range(2)]
    dt = time.perf_counter() - ta
    out = base_line(args, updates / (ms * 1e-3), ms, 1, "u8 categories, f32 logits")
    cfg = workload_config(args)
    cfg["block_kernels"] = kinds
    out.update({"config": cfg, "gpu_launches": args.steps * 2,
                "roofline": hbm_roofline(updates / 2, 7.0 + 6.0 * K * K * 4 / chains, ms / 2, "k_cat_warp" if all(k == 5 for k in kinds) and K <= 16 and chains >= 128 else "k_cat_generic",
                                         note="gather of six neighbour bytes and six K x K weight rows per node; instruction-issue bound"),
                "e2e": {"value": updates * args.steps / dt, "unit": UNIT, "h2d_bytes_per_step": chains * n / args.steps, "d2h_bytes_per_step": chains * n / args.steps, "seconds": dt,
                        "call": "thrml_state_upload_u8_many + thrml_run_blocks + thrml_state_download_u8"}})
    del back
    if not args.no_cpu_baseline:
        out["cpu_baseline"], _ = cpu_baseline(args, os.cpu_count() or 1)
    return out


def run_mixed(T, torch, args, rank, world, device, dist, ctx, comm):
    """Spin / K-state checkerboard with three-spin terms (workloads.spin_category_checkerboard): two spin blocks whose slots have
    categorical tails and spin-pair tails (k_spin_wide) and one categorical block with spin tails (k_cat_warp).  Not a
    configuration of the reference's benchmark list: it measures the kernels that serve general factor structures."""
    from thrml_rs_b200 import workloads as W
    side, K, chains = args.side, 4, args.chains
    model = W.spin_category_checkerboard(side, K)
    n = model["n"]
    program = T.Program(W.fill_factors(T.Builder(model["kinds"], model["dtype_order"]), model, ctx=ctx), ctx)
    kinds = [program.block_kernel(b) for b in range(3)]
    names = {0: "k_spin_generic", 2: "k_cat_generic", 5: "k_cat_warp", 7: "k_spin_wide", 8: "k_cat_many"}
    state = T.ChainState(program, chains)
    state.randomize(5)
    stream = torch.cuda.ExternalStream(ctx.stream)

    def sync():
        ctx.synchronize()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        state.sample_blocks(i)
    sampler = ClockSampler(device)
    t0 = time.time()
    ms = timed(torch, stream, lambda: [state.sample_blocks(100 + i) for i in range(args.steps)], sync) / args.steps
    clocks = sampler.stop(t0, time.time())
    # each block's kernel alone.  Algorithmic bytes per update: one byte per tail read and one written, plus the node's slot
    # parameters (position, weight row) amortised over the chains
    tails = [4 + 2, 4, 4]          # spins of even rows: four categorical neighbours and the spin pair of the three-spin term
    params = [5 * 8 + 4 * 4 * K + 8, 4 * 8 + 4 * 4 * K + 4, 4 * 8 + 4 * 4 * K + 4 * K]
    per_block = []
    for b in range(3):
        nb = len(model["blocks"][b])
        bms = timed(torch, stream, lambda: [state.sample_single_block(b, 7 + i) for i in range(10)], sync) / 10
        per_block.append({"block": b, "kernel": names.get(kinds[b], str(kinds[b])), "nodes": int(nb), "ms": bms, "site_updates_per_s": nb * chains / (bms * 1e-3),
                          "bytes_per_update": tails[b] + 1 + params[b] / chains})
    top = max(per_block, key=lambda r: r["ms"])
    updates = float(n) * chains
    rng = np.random.default_rng(9)
    host = [pinned(torch, rng.integers(0, 2 if b < 2 else K, (chains, len(model["blocks"][b])), dtype=np.uint8)) for b in range(3)]
    sync()
    ta = time.perf_counter()
    state.upload_many([0, 1, 2], [h.numpy() for h in host])
    state.run_blocks(55, args.steps)
    back = [state.download(b, np.uint8) for b in range(3)]
    dt = time.perf_counter() - ta
    del back
    out = base_line(args, updates / (ms * 1e-3), ms, 1, "u8 spins and categories, f32 fields and logits")
    cfg = workload_config(args)
    cfg["block_kernels"] = kinds
    out.update({"config": cfg, "clocks": clocks, "gpu_launches": args.steps * 2, "per_block": per_block,
                "roofline": hbm_roofline(top["nodes"] * float(chains), top["bytes_per_update"], top["ms"], top["kernel"],
                                         note="the block that takes the most time; per_block lists all three"),
                "e2e": {"value": updates * args.steps / dt, "unit": UNIT, "h2d_bytes_per_step": chains * n / args.steps, "d2h_bytes_per_step": chains * n / args.steps, "seconds": dt,
                        "call": "thrml_state_upload_u8_many + thrml_run_blocks + thrml_state_download_u8"}})
    if not args.no_cpu_baseline:
        out["cpu_baseline"], _ = cpu_baseline(args, os.cpu_count() or 1)
        if not args.no_parity:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import fullsize_checks as F
            from oracle import oracle as O
            out["parity_check"] = F.mixed_check(T, O, model, program, state, chains, threads=os.cpu_count() or 1)
    return out


def run_potts(T, torch, args, rank, world, device, dist, ctx, comm):
    """Categorical (Potts-like) EBM on a 128^3 periodic lattice, K = 10, three direction tables N(0, 0.3^2), unary terms
    N(0, 0.1^2), beta = 1, 1024 chains, Gumbel-argmax updates, category marginals observed every sweep."""
    from thrml_rs_b200 import potts
    side, K, chains = args.side, 10, args.chains
    n = side ** 3
    tables, unary = potts_arrays(side, K)
    # chains are independent: with several GPUs every rank holds `chains` of them (global ids rank * chains + c, so the draws
    # do not depend on the sharding) and the category counts are added over the ranks by one allreduce inside the timed region
    lat = potts.PottsLattice(side, side, side, K, tables, unary, 1.0, chains, rank * chains, ctx)
    lat.randomize(5)
    stream = torch.cuda.ExternalStream(ctx.stream)

    def sync():
        ctx.synchronize()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()

    def step(i):  # one sweep followed by the marginal observation, as one schedule of the library's driver (the second colour's
        lat.sample_with_marginals(300 + i, 1, 1, 1)  # update and the first's count the categories they draw)

    def steps_and_reduce():
        for i in range(args.steps):
            step(100 + i)
        if comm:
            lat.allreduce_marginals(comm)

    for i in range(max(args.warmup, 3)):
        step(i)
    if comm:  # the communicator's first large collective, outside the timed region; the counts start again afterwards
        lat.allreduce_marginals(comm)
    lat.reset_marginals()
    sampler = ClockSampler(device) if rank == 0 else None
    t0 = time.time()
    ms = max_over_ranks(torch, dist, timed(torch, stream, steps_and_reduce, sync)) / args.steps
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if sampler else None
    counts, n_obs = lat.read_marginals()
    update_ms = timed(torch, stream, lambda: lat.run_blocks(9, 4), sync) / 8  # one colour update, without the observer
    updates = float(n) * chains * world
    out = base_line(args, updates / (ms * 1e-3), ms, world, "u8 categories, f32 logits")
    out.update({"config": workload_config(args, world=world), "clocks": clocks, "gpu_launches": args.steps * 2 + (1 if comm else 0),
                "roofline": hbm_roofline(float(n) * chains / 2, 2 + 120.0 / chains, update_ms, "k_potts_update",
                                         note="instruction-bound by construction: a Gumbel draw (two logarithms, a 23-bit uniform) per category and update",
                                         dram_bytes_per_update=POTTS_DRAM_BYTES_PER_UPDATE if (K, chains) == (10, 1024) else None,
                                         dram_provenance="ncu dram__bytes_read.sum + dram__bytes_write.sum of one k_potts_update launch on a 64^3 lattice, 1024 chains "
                                                         "(profiles/k_potts_update_potts128.md), scaled by site updates"),
                "marginal_check": {"observations_per_node": int(n_obs), "rows_sum_to_observations": bool(np.all(counts.sum(axis=1) == n_obs))}})
    del counts
    if world > 1:
        return out
    if not args.no_e2e:
        # end to end: initial categories from pinned host memory, the schedule (0 warm-up, steps + 1 samples, 1 sweep each) with
        # the marginal observer inside the library, counts read back
        rng = np.random.default_rng(9)
        host = pinned(torch, rng.integers(0, K, (chains, n), dtype=np.uint8))
        sync()
        ta = time.perf_counter()
        lat.upload(host.numpy())
        lat.sample_with_marginals(41, 0, args.steps + 1, 1)
        lat.read_marginals()
        dt = time.perf_counter() - ta
        out["e2e"] = {"value": updates * args.steps / dt, "unit": UNIT, "h2d_bytes_per_step": chains * n / args.steps, "d2h_bytes_per_step": n * K * 4 / args.steps, "seconds": dt,
                      "call": "thrml_potts_upload (pinned host bytes) + thrml_potts_sample_with_marginals + thrml_potts_read_marginals"}
        del host
    if not args.no_cpu_baseline:
        out["cpu_baseline"], _ = cpu_baseline(args, os.cpu_count() or 1)
    if not args.no_parity:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import fullsize_checks as F
        from oracle import oracle as O
        del lat
        out["parity_check"] = F.potts_check(T, O, side=min(side, 64), K=K, chains=chains, ctx=ctx)
    return out


# -----------------------------------------------------------------------------------------------------------
# One huge bit-packed lattice, rows sharded over the GPUs.
# -----------------------------------------------------------------------------------------------------------
def run_lattice(T, torch, args, rank, world, device, dist, ctx, comm):
    """One large periodic 2-D Ising lattice (J = 0.4407, zero bias, beta = 1), bit-packed, 16 chains, checkerboard blocks,
    sharded by row stripes over the GPUs with a one-row halo exchange per half-sweep (grouped ncclSend / ncclRecv inside
    thrml_lattice_run_blocks); magnetisation and energy are recorded on the device after every sweep and reduced to
    their first and second moments at the end.  Strong scaling: the lattice is fixed, the stripes shrink."""
    from thrml_rs_b200 import lattice
    side, chains = args.side, args.chains
    lat = lattice.DistributedStripe(side, side, 0.4407, 0.0, 1.0, chains, comm, ctx)
    lat.randomize(11)
    stream = torch.cuda.ExternalStream(ctx.stream)

    def sync():
        ctx.synchronize()
        torch.cuda.synchronize()
        if dist:
            dist.barrier()

    lat.run_blocks(50, max(args.warmup, 3), record=True)
    lat.moments()  # the read-out collective once, outside the timed region
    lat.series_reset()
    sampler = ClockSampler(device) if rank == 0 else None
    t0 = time.time()
    ms = max_over_ranks(torch, dist, timed(torch, stream, lambda: lat.run_blocks(99, args.steps, record=True), sync))
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if sampler else None
    mom, n_rec = lat.moments()
    n_spins = float(side) * side
    updates = n_spins * chains * args.steps
    out = base_line(args, updates / (ms * 1e-3), ms / args.steps, world, "1-bit spins, u32 thresholds", scaling="strong")
    out.update({"config": workload_config(args, world=world), "clocks": clocks,
                "gpu_launches": args.steps * (3 if world == 1 else 7),  # per sweep: two colour updates (boundary rows apart when striped) and the observable kernel
                "roofline": hbm_roofline(n_spins * chains / 2 / world, 0.25, ms / args.steps / 2, "k_lattice_update_sliced",
                                         note="0.25 B per update: this kernel is bound by instruction issue (8.6 instructions per update: noise planes, bit-sliced compare), not by HBM; "
                                              "launch_ms is half a sweep, halo exchange and observable recording included",
                                         dram_bytes_per_update=LATTICE_DRAM_BYTES_PER_UPDATE if chains == 16 else None,
                                         dram_provenance="ncu dram__bytes_read.sum + dram__bytes_write.sum of one k_lattice_update_sliced launch on a 16384^2 lattice, 16 chains "
                                                         "(profiles/k_lattice_update_sliced_ising_bitpacked.md), scaled by site updates"),
                "observables": {"records": int(n_rec), "m_mean": float(np.mean(mom[0])), "m2_mean": float(np.mean(mom[1])), "e_mean": float(np.mean(mom[2])), "e2_mean": float(np.mean(mom[3]))}})
    if not args.no_e2e:
        # end to end: this rank's rows of the initial state from pinned host memory as bits, the sweeps with the observable
        # series, the moments read back
        rng = np.random.default_rng(21 + rank)
        rows = side // world
        host = pinned_u32(torch, rng.integers(0, 1 << 32, (chains, rows, side // 32), dtype=np.uint32))
        sync()
        ta = time.perf_counter()
        lat.series_reset()
        lat.upload_bits(host.numpy().view(np.uint32))
        lat.run_blocks(123, args.steps, record=True)
        lat.moments()
        dt = max_over_ranks(torch, dist, time.perf_counter() - ta)
        out["e2e"] = {"value": updates / dt, "unit": UNIT, "h2d_bytes_per_step": world * host.numel() * 4 / args.steps, "d2h_bytes_per_step": 2 * chains * 8, "seconds": dt,
                      "call": "thrml_lattice_upload_bits (pinned host bits) + thrml_lattice_run_blocks(record) + thrml_lattice_moments"}
        del host
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            out["cpu_baseline"], _ = cpu_baseline(args, os.cpu_count() or 1)
        if not args.no_parity:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import fullsize_checks as F
            from oracle import oracle as O
            del lat
            out["parity_check"] = F.lattice_check(T, O, side=min(side, 2048), chains=chains, ctx=ctx)
    return out


if __name__ == "__main__":
    main()
