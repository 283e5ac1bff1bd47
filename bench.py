"""Benchmark of the hot path: sampled dt-steps of a PaiNN/meanflow denoiser (radius graph rebuilt
every step -> fused message kernels -> channel mixing), reported as edge-messages/s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One process per GPU (torchrun for N > 1); systems are sharded across ranks, nothing crosses GPUs
inside a step, one NCCL gather of the final positions at the end of the timed region."""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "learned-dynamics_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402

WORKLOADS = {
    # benchmark config 3: periodic dense-system rollout, graph rebuilt every step
    "periodic_rollout_16x8192": dict(systems=16, nodes=8192, box=20.0, cutoff=4.0, n=128, n_rbf=8, radial="gaussian",
                                     blks=(1, 3), ntypes=4, sigma0=0.05, kind="periodic"),
    # benchmark config 4 geometry (open polymers) with the PaiNN denoiser
    "polymers_1024x256": dict(systems=1024, nodes=256, box=None, cutoff=5.0, n=128, n_rbf=16, radial="gaussian",
                              blks=(2, 4), ntypes=20, sigma0=0.05, kind="polymer"),
    # small case for smoke runs and profiler captures
    "periodic_small_4x2048": dict(systems=4, nodes=2048, box=12.6, cutoff=4.0, n=128, n_rbf=8, radial="gaussian",
                                  blks=(1, 3), ntypes=4, sigma0=0.05, kind="periodic"),
}
# benchmark configs 4 and 2 with the l<=2 (scalar / vector / rank-2) denoiser: 6 layers, (128, 64, 32) channels,
# 128 product channels, cutoff 5.0, 20 bead types; radial read-in = the reference's 8 Jacobi functions
WORKLOADS["polymers_l2_1024x256"] = dict(systems=1024, nodes=256, box=None, cutoff=5.0, model="bee", dims=(128, 64, 32, 128),
                                         depth=6, ntypes=20, sigma0=0.05, kind="polymer")
WORKLOADS["polymers_l2_64x512"] = dict(systems=64, nodes=512, box=None, cutoff=5.0, model="bee", dims=(128, 64, 32, 128),
                                       depth=6, ntypes=20, sigma0=0.05, kind="polymer")
# benchmark config 1: neighbour graph only (handled by run_graph_bench)
WORKLOADS["proxattn_32x4096_d64"] = dict(proxattn=True, Z=32, N=4096, dim=64)
WORKLOADS["proxattn_32x4096_d128"] = dict(proxattn=True, Z=32, N=4096, dim=128)
WORKLOADS["graph_32x4096"] = dict(systems=32, nodes=4096, box=16.0, cutoff=2.5, kind="periodic", graph_only=True)
# The metric (edge-messages/s and dt-steps/s at 1/2/4/8 GPUs) is quoted on benchmark config 4: 1024 polymers x 256 beads,
# the 6-layer (128, 64, 32) denoiser, sharded by system.
DEFAULT_WORKLOAD = "polymers_l2_1024x256"
# DRAM bytes per processed edge of the dominant kernel, from the committed profiler captures of a smaller case
# (profiles/): read + write bytes of one launch / its edge count. Traffic is dominated by per-edge inputs (rij, dst)
# and by one pass over the node features, both proportional to the edge count at fixed degree.
DRAM_BYTES_PER_EDGE = {"bee_scalar_tc_kernel": 83.0, "bee_vd_kernel": 200.4, "bee_vd_tc_kernel": 208.0, "bee_fused_tc_kernel": 217.2,
                       "painn_message_tc_kernel": 33.8}
# timer regions of the edge kernels of an l<=2 message layer -> kernel names
BEE_EDGE_REGIONS = {"bee_messages_fused_tc": "bee_fused_tc_kernel", "bee_messages_scalar_tc": "bee_scalar_tc_kernel",
                    "bee_messages_scalar": "bee_scalar_kernel", "bee_messages_vd": "bee_vd_kernel",
                    "bee_messages_vd_tc": "bee_vd_tc_kernel"}


def make_positions(w, systems, seed):
    g = torch.Generator().manual_seed(seed)
    if w["kind"] == "periodic":
        return torch.rand(systems, w["nodes"], 3, generator=g) * w["box"]
    return torch.cumsum(torch.randn(systems, w["nodes"], 3, generator=g) / 3 ** 0.5, dim=1)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return d["hbm_gbs"], d["bf16_tflops"], d["bf16_tflops_sustained"], "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled during the timed region."""

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def start(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        mx = [int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [nm for k, nm in enumerate(names) if any(len(r) > 2 + k and r[2 + k] == "Active" for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm)}


def message_flops_per_edge(n, n_rbf):
    """distance MLP (n_rbf -> 4n -> 4n -> 4n) per edge"""
    return 2 * (n_rbf * 4 * n + 2 * (4 * n) ** 2)


def build_model(w, device):
    from ld_b200 import painn
    torch.manual_seed(1234)
    if w.get("model") == "bee":
        from ld_b200 import bee
        dn = bee.BeeDenoiser(w["cutoff"], *w["dims"], ntypes=w["ntypes"], depth=w["depth"]).to(device)
        with torch.no_grad():
            dn.readout.W.mul_(1e-3)  # small velocity read-out: a random-init rollout stays in the input distribution
        return dn
    dn = painn.SE3ITO(w["cutoff"], w["n"], w["nodes"], w["ntypes"], w["blks"][0], w["blks"][1], n_rbf=w["n_rbf"],
                      radial=w["radial"]).to(device)
    return dn


def cpu_reference_rate(w, threads, budget_nodes=1024, steps=1):
    """The reference's PyTorch formulation on the host cores (oracle restatement), on a bounded
    sample: one system at the workload's density with `budget_nodes` nodes. Returns
    (edge-messages/s, description)."""
    from oracle import reference_math as R
    torch.set_num_threads(threads)
    nodes = min(budget_nodes, w["nodes"])
    torch.manual_seed(1234)
    if w.get("model") == "bee":
        systems = max(1, budget_nodes // w["nodes"])
        dn = R.OBeeDenoiser(w["cutoff"], *w["dims"], ntypes=w["ntypes"], depth=w["depth"])
        with torch.no_grad():
            dn.readout.W.mul_(1e-3)
        g = torch.Generator().manual_seed(4321)
        x = torch.cumsum(torch.randn(systems, w["nodes"], 3, generator=g) / 3 ** 0.5, dim=1)
        types = torch.randint(0, w["ntypes"], (w["nodes"],), generator=g)
        edges, t0 = 0, time.perf_counter()
        for _ in range(steps):
            x = dn.generate(x, torch.randn(x.shape, generator=g), w["sigma0"], None, types)
            edges += dn.edges_last
        dt = time.perf_counter() - t0
        return edges / dt, f"{systems} system(s) x {w['nodes']} nodes, {steps} step(s), {edges} edge-messages in {dt:.1f} s"
    dn = R.OSE3ITO(w["cutoff"], w["n"], nodes, w["ntypes"], w["blks"][0], w["blks"][1], w["n_rbf"], w["radial"])
    g = torch.Generator().manual_seed(4321)
    if w["kind"] == "periodic":
        box_len = w["box"] * (nodes / w["nodes"]) ** (1.0 / 3.0)
        box = (box_len,) * 3
        x = torch.rand(1, nodes, 3, generator=g) * box_len
        bs = bd = torch.zeros(0, dtype=torch.int64)
    else:
        box = None
        x = torch.cumsum(torch.randn(1, nodes, 3, generator=g) / 3 ** 0.5, dim=1)
        bs, bd = R.chain_bonds(1, nodes)
    types = torch.randint(0, w["ntypes"], (nodes,), generator=g)
    edges, t0 = 0, time.perf_counter()
    for _ in range(steps):
        noise = torch.randn(1, nodes, 3, generator=g)
        x = R.meanflow_generate(dn, x, noise, w["sigma0"], box, types, bs, bd)
        edges += dn.edges_last
    dt = time.perf_counter() - t0
    desc = f"1 system x {nodes} nodes at the workload's density, {steps} step(s), {edges} edge-messages in {dt:.1f} s"
    return edges / dt, desc


def workload_config(name, w):
    """the static description of a workload; the same dict in both arms' JSON lines"""
    is_bee = w.get("model") == "bee"
    cfg = {"workload": name, "systems": w["systems"], "nodes_per_system": w["nodes"], "cutoff": w["cutoff"],
           "width": list(w["dims"]) if is_bee else w["n"], "radial_basis": 8 if is_bee else w["n_rbf"],
           "message_layers_per_step": w["depth"] if is_bee else 2 * sum(w["blks"]),
           "graph_rebuilds_per_step": 1 if is_bee else 2,
           "l2_policy": "inputs larger than L2 (per-step node features and gathers exceed 126 MB)"}
    if is_bee:
        # the benchmark text asks for 16 radial basis functions; the reference's l<=2 layer reads the edge length in
        # through its eight polynomial functions (managan/jacobi_radenc.py:27-37), and that layer is what is built
        cfg["radial_basis_baseline"] = 16
        cfg["radial_basis_note"] = "the reference's Messages layer has 8 polynomial radial functions; 16 is the benchmark text"
    return cfg


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    threads = len(os.sched_getaffinity(0))
    rates = []
    desc = ""
    for i in range(args.warmup + args.steps):
        r, desc = cpu_reference_rate(w, threads, budget_nodes=args.cpu_nodes)
        if i >= args.warmup:
            rates.append(r)
    value = sum(rates) / len(rates)
    line = {
        "impl": "reference", "metric": "edge_messages_per_sec", "value": value, "unit": "edge-messages/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload, w),
        "note": "reference's PyTorch formulation (CPU oracle restatement) on host cores, bounded sample of the workload",
        "cpu_baseline": {"value": value, "unit": "edge-messages/s", "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "edge-messages/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def bee_layer_roofline(w, ktimes, local_edges, systems_local, tc_path, hbm, tf_sus, how):
    """Roofline of the fused gather -> product -> per-node sum of one l<=2 message layer: all edge kernels of a layer
    together against the algorithmic bytes of the layer (every edge pulls the 13*chan float32 values of its neighbour
    plus (src, dst, r_ij); outputs a + 3v + 9d floats once per node)."""
    da, dv, dd, ch = w["dims"]
    regions = {r: ktimes[r] for r in BEE_EDGE_REGIONS if r in ktimes and ktimes[r]["launches"]}
    if not regions:
        return None
    layers = max(v["launches"] for v in regions.values())          # one launch of each edge kernel per layer
    layer_s = sum(v["ms"] for v in regions.values()) * 1e-3 / layers
    edges_layer = local_edges / layers                              # rank 0's own launches
    nodes_layer = systems_local * w["nodes"]
    alg_bytes = edges_layer * (20 + 4 * 13 * ch) + nodes_layer * 4 * (da + 3 * dv + 9 * dd)
    flops = 2 * (3 * ch * da + 9 * da * da) * edges_layer           # per-edge Y map + mlp_a
    achieved = alg_bytes / layer_s / 1e9
    traffic = sum(DRAM_BYTES_PER_EDGE.get(BEE_EDGE_REGIONS[r], 0.0) for r in regions) * edges_layer
    known = all(BEE_EDGE_REGIONS[r] in DRAM_BYTES_PER_EDGE for r in regions)
    return {"bound": "hbm", "kernel": "l<=2 message layer: " + " + ".join(BEE_EDGE_REGIONS[r] for r in regions),
            "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
            "traffic": traffic if known else None, "achieved_dram_gbs": traffic / layer_s / 1e9 if known else None,
            "peak_source": f"hbm_gbs, {how}", "layers": layers, "avg_layer_ms": layer_s * 1e3,
            "algorithmic_bytes_per_layer": alg_bytes,
            "kernels": {BEE_EDGE_REGIONS[r]: {"avg_launch_ms": v["ms"] / v["launches"], "launches": v["launches"]} for r, v in regions.items()},
            "tensor_tflops": flops / layer_s / 1e12 if tc_path else None,
            "tensor_frac_of_sustained_bf16": flops / layer_s / 1e12 / tf_sus if tc_path else None,
            "note": "achieved = algorithmic bytes of the layer / time of all its edge kernels; the gathered rows are read as BF16 "
                    "and almost always from L2 (all blocks walk the node range in segments), so the DRAM traffic ('traffic', "
                    "'achieved_dram_gbs', from the profiler capture of a smaller case scaled by edges) is a small part of the "
                    "algorithmic bytes: the kernels are bound by shared-memory bandwidth and instruction issue, not by HBM"}


def run_graph_bench(args, w):
    """Radius graph only (benchmark config 1): count + fill per step at a fixed capacity, no host sync."""
    from ld_b200 import graph as G
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    box = (w["box"],) * 3
    pos = make_positions(w, w["systems"], seed=1001).to(dev)
    builder = G.RadiusGraphBuilder(w["systems"], w["nodes"], w["cutoff"], box, device=dev)
    g = builder.build(pos, want_shift=True, want_rij=False)
    E, Nt = g["E"], w["systems"] * w["nodes"]
    src, dst, shift = torch.empty_like(g["src"]), torch.empty_like(g["dst"]), torch.empty_like(g["shift"])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # larger than L2

    def step():
        builder.build_fixed(pos, E, src, dst, shift, None)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    total_ms = 0.0
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1)
    # a build takes well under a millisecond: keep the same kernels running (untimed) until the clock sampler has
    # a few readings under load
    t_end = time.perf_counter() + 0.8
    while len(sampler.rows) < 4 and time.perf_counter() < t_end:
        for _ in range(50):
            step()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    assert int(builder.status.item()) == 0 and torch.equal(dst, g["dst"])
    # end to end: host positions in, edge list out
    pos_host = pos.cpu().pin_memory()
    out_host = torch.empty(3 * E, dtype=torch.int32).pin_memory()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(args.steps):
        p = pos_host.to(dev, non_blocking=True)
        builder.build_fixed(p, E, src, dst, shift, None)
        out_host[:E].copy_(src, non_blocking=True); out_host[E:2 * E].copy_(dst, non_blocking=True)
        out_host[2 * E:].copy_(shift, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1)
    hbm, _, _, how = peaks()
    ms = total_ms / args.steps
    alg_bytes = 12 * Nt + 4 * (Nt + 1) + 12 * E   # positions in, CSR offsets, (src, dst, packed shift) out
    achieved = alg_bytes / (ms * 1e-3) / 1e9
    line = {
        "metric": "graph_edges_per_sec", "value": E / (ms * 1e-3), "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32/int32", "data": "synthetic",
        "config": {"workload": args.workload, "systems": w["systems"], "nodes_per_system": w["nodes"], "box": w["box"],
                   "cutoff": w["cutoff"], "edges": E, "l2_policy": "256 MB flush buffer written between timed iterations"},
        "e2e": {"value": E * args.steps / (e2e_ms * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": Nt * 12, "d2h_bytes_per_step": 12 * E},
        "gpu_launches": 14 * args.steps, "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "radius graph build (13 kernels; neighbour_kernel<0/1> dominate)", "achieved": achieved,
                     "peak": hbm, "unit": "GB/s", "frac": achieved / hbm, "traffic": None, "peak_source": f"hbm_gbs, {how}"},
    }
    if not args.no_cpu_baseline:
        from oracle import reference_math as R
        t = time.perf_counter()
        o = R.radius_graph(pos[:1].cpu(), w["cutoff"], box)
        dt = time.perf_counter() - t
        line["cpu_baseline"] = {"value": o["E"] / dt, "unit": "edges/s", "cores": 1, "kind": "port",
                                "sample": f"1 system x {w['nodes']} particles, brute force over all pairs, {o['E']} edges in {dt:.1f} s"}
    print(json.dumps(line))


def run_proxattn_bench(args, w):
    """Dense proximity attention (forward and backward device time) on one GPU."""
    from ld_b200 import proxattn as PA
    Z, N, dim, heads, reps = w["Z"], w["N"], w["dim"], 4, max(args.steps, 1)
    g = torch.Generator().manual_seed(0)
    q, k, v, d_out = (torch.randn(Z, N, dim, generator=g).cuda() for _ in range(4))
    x, y = (4 * torch.rand(Z, N, 3, generator=g)).cuda(), (4 * torch.rand(Z, N, 3, generator=g)).cuda()
    r0sq = (0.2 + torch.rand(heads, generator=g)).cuda()
    ins = [t.requires_grad_(True) for t in (q, k, v, x, y)]
    out = {}
    for periodic in (False, True):
        box = (4.0, 4.0, 4.0) if periodic else None
        for precision in ("fp32", "tf32"):
            for backward in (False, True):
                if backward and precision == "tf32":
                    continue
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                res = PA._ProxAttn.apply(*ins, r0sq, box, precision)
                for i in range(reps + max(args.warmup, 1)):
                    if i == max(args.warmup, 1):
                        e0.record()
                    if backward:
                        torch.autograd.grad(res, ins, d_out, retain_graph=True)
                    else:
                        res = PA._ProxAttn.apply(*ins, r0sq, box, precision)
                e1.record()
                torch.cuda.synchronize()
                out[f"{'periodic' if periodic else 'open'}_{precision}_{'bwd' if backward else 'fwd'}_ms"] = e0.elapsed_time(e1) / reps
    pair_flops = 2.0 * Z * N * N * dim
    ms = out["open_tf32_fwd_ms"]
    print(json.dumps({"metric": "proxattn_forward_tflops", "value": 2 * pair_flops / ms * 1e-9, "unit": "TFLOP/s", "n_gpus": 1,
                      "steps": reps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "tf32",
                      "data": "synthetic", "config": {"workload": args.workload, "Z": Z, "N": N, "dim": dim},
                      "times_ms": {k_: round(v_, 4) for k_, v_ in out.items()},
                      "fp32_forward_tflops": 2 * pair_flops / out["open_fp32_fwd_ms"] * 1e-9,
                      "fp32_backward_tflops": 7 * pair_flops / out["open_fp32_bwd_ms"] * 1e-9}))


def positions_checksum(x):
    """order-independent-of-ranks fingerprint of a position tensor: sha256 of its float32 bytes (first 16 hex digits)"""
    import hashlib
    return hashlib.sha256(x.detach().cpu().contiguous().numpy().tobytes()).hexdigest()[:16]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32"],
                    help="bf16: per-edge MLP on tcgen05 (2e-2 parity); fp32: SIMT path (1e-5 parity)")
    ap.add_argument("--cpu-nodes", type=int, default=3072,
                    help="nodes of the bounded CPU-baseline sample (10-30 s of host work)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fp32-leg", action="store_true", help="skip the two float32 steps reported under 'fp32'")
    ap.add_argument("--l2-layer", default="pair", choices=["pair", "single"],
                    help="l<=2 message layer: 'pair' = two edge kernels (default), 'single' = one edge kernel per layer "
                         "(chan = dim_a = 128; per-node sums accumulated in tensor memory; measured slower)")
    ap.add_argument("--product-sums", default="fma", choices=["fma", "tensor"],
                    help="l<=2 network: rank-1 / rank-2 product sums by FP32 FMAs (default) or by one tcgen05 MMA per edge")
    ap.add_argument("--component-major", action="store_true",
                    help="keep the vector / rank-2 node features as [.., 3|9, chan] between the layers (plain-row channel mixings)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if w.get("graph_only") or w.get("proxattn"):
        if rank == 0:
            (run_graph_bench if w.get("graph_only") else run_proxattn_bench)(args, w)
        return
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return

    import torch.distributed as dist
    from ld_b200 import painn, ops
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ld_b200 import sharding
    sys_begin, sys_end = sharding.shard_range(w["systems"], rank, world)
    per = sys_end - sys_begin
    box = None if w["box"] is None else (w["box"],) * 3

    is_bee = w.get("model") == "bee"
    if is_bee:
        from ld_b200 import bee
        dn = bee.set_precision(build_model(w, dev), args.precision)
        dn.component_major = args.component_major
        for m in dn.modules():
            if isinstance(m, bee.Messages):
                m.fused_kernel = args.l2_layer == "single"
                m.vd_tensor_core = args.product_sums == "tensor"
    else:
        dn = painn.set_precision(build_model(w, dev), args.precision)
    painn.enable_rollout_graphs(dn)   # fixed-capacity graph buffers: no step waits for its edge count
    types = torch.randint(0, w["ntypes"], (w["nodes"],), generator=torch.Generator().manual_seed(99)).to(dev)
    if not is_bee:
        bond = painn.chain_bond_graph(per, w["nodes"], dev) if w["kind"] == "polymer" else painn.empty_bond_graph(per, w["nodes"], dev)
        mf = painn.Meanflow(dn, box, w["sigma0"], types, bond)
    x_all = make_positions(w, w["systems"], seed=1003)
    x_host = x_all[sys_begin:sys_end].contiguous().pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    counter = torch.zeros(1, dtype=torch.int64, device=dev)
    NOISE_SEED = 777

    def device_step(x, step):
        # counter-based noise keyed by (global system, step): the rollout does not depend on the number of ranks
        noise = sharding.shard_noise(tuple(x.shape), sys_begin, NOISE_SEED, step, dev)
        if is_bee:
            return dn.generate(x, noise, w["sigma0"], box, types, counter)
        return mf.generate(x, noise, counter)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_rollout(steps, warmup):
        """device-resident rollout: returns (ms, total edges over ranks, rank-local edges, per-kernel times, final positions)"""
        x = x_host.to(dev)
        for s_ in range(warmup):
            x = device_step(x, s_)
        sharding.gather_positions(x, w["systems"])  # untimed: the first collective also sets up the NCCL communicator
        barrier()
        counter.zero_()
        ops.KERNEL_TIMER.reset(enabled=True)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for s_ in range(steps):
            x = device_step(x, warmup + s_)
        final = sharding.gather_positions(x, w["systems"])  # the one collective of a rollout (NCCL over NVLink)
        e1.record()
        barrier()
        painn.finish_rollout_graphs(dn)
        ops.check_tc_status(dev)
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        edges = counter.clone()
        local_edges = int(counter.item())
        ktimes = ops.KERNEL_TIMER.summary()
        launches = ops.KERNEL_TIMER.total_launches
        ops.KERNEL_TIMER.reset(enabled=False)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(edges, op=dist.ReduceOp.SUM)
        return ms.item(), int(edges.item()), local_edges, ktimes, launches, final

    # ---- device-resident timing ------------------------------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    total_ms, total_edges, local_edges, ktimes, launches, final = timed_rollout(args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end through the public API with host buffers ---------------------------------------
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    counter.zero_()
    barrier()
    t0.record()
    for s_ in range(args.steps):
        xd = x_host.to(dev, non_blocking=True)
        xd = device_step(xd, 1000 + s_)
        out_host.copy_(xd, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        x_host.copy_(out_host)
    t1.record()
    barrier()
    ms2 = torch.tensor([t0.elapsed_time(t1)], device=dev)
    edges2 = counter.clone()
    if world > 1:
        dist.all_reduce(ms2, op=dist.ReduceOp.MAX)
        dist.all_reduce(edges2, op=dist.ReduceOp.SUM)
    x_host.copy_(x_all[sys_begin:sys_end])

    # ---- the float32 path (the reference's own precision), two timed steps ---------------------------
    fp32 = None
    if is_bee and args.precision == "bf16" and not args.no_fp32_leg:
        bee.set_precision(dn, "fp32")
        f_ms, f_edges, f_local, f_k, _, f_final = timed_rollout(2, 1)
        bee.set_precision(dn, "bf16")
        fp32 = {"ms": f_ms, "edges": f_edges, "local_edges": f_local, "ktimes": f_k, "final": f_final}

    if rank == 0:
        hbm, tf_burst, tf_sus, how = peaks()
        value = total_edges / (total_ms * 1e-3)
        e2e_value = int(edges2.item()) / (ms2.item() * 1e-3)
        tc_path = args.precision == "bf16"
        roof = None
        if is_bee:
            roof = bee_layer_roofline(w, ktimes, local_edges, per, tc_path, hbm, tf_sus, how)
        else:
            kname = "painn_message_tc_kernel" if tc_path else "painn_message_kernel"
            msg = ktimes.get("painn_message_tc" if tc_path else "painn_message", {"launches": 0, "ms": 0.0})
            flops = message_flops_per_edge(w["n"], w["n_rbf"])
            if msg["launches"]:
                per_launch_s = msg["ms"] * 1e-3 / msg["launches"]
                edges_launch = local_edges / msg["launches"]
                achieved = flops * edges_launch / per_launch_s / 1e12
                roof = {"bound": "tensor", "kernel": kname, "achieved": achieved, "peak": tf_sus, "unit": "TFLOP/s",
                        "frac": achieved / tf_sus,
                        "traffic": DRAM_BYTES_PER_EDGE[kname] * edges_launch if kname in DRAM_BYTES_PER_EDGE else None,
                        "peak_source": f"bf16_tflops_sustained, {how}", "launches": msg["launches"], "avg_launch_ms": per_launch_s * 1e3,
                        "note": ("tcgen05 BF16 MMAs of the per-edge distance MLP (algorithmic flops: 2*(n_rbf*4n + 2*(4n)^2) per edge)"
                                 if tc_path else "FP32 SIMT arithmetic measured against the dense bf16 tensor peak")}
        line = {
            "metric": "edge_messages_per_sec", "value": value, "unit": "edge-messages/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16" if tc_path else "f32", "data": "synthetic",
            "config": workload_config(args.workload, w), "precision": args.precision, "l2_layer": args.l2_layer if is_bee else None, "product_sums": args.product_sums if is_bee else None,
            "edges_per_step": total_edges // args.steps,
            "dt_steps_per_sec": args.steps / (total_ms * 1e-3),
            "system_steps_per_sec": args.steps * w["systems"] / (total_ms * 1e-3),
            "e2e": {"value": e2e_value, "unit": "edge-messages/s", "h2d_bytes_per_step": x_host.numel() * 4 * world,
                    "d2h_bytes_per_step": out_host.numel() * 4 * world, "ms_per_step": ms2.item() / args.steps},
            "gpu_launches": launches,
            "kernel_ms": {k: round(v["ms"], 3) for k, v in ktimes.items()},
            "clocks": clocks, "roofline": roof,
            # sha256 of the gathered final positions: identical at 1, 2, 4 and 8 GPUs (noise keyed by system and step)
            "final_checksum": positions_checksum(final),
        }
        if fp32 is not None:
            line["fp32"] = {"value": fp32["edges"] / (fp32["ms"] * 1e-3), "unit": "edge-messages/s", "steps": 2, "warmup": 1,
                            "ms_per_step": fp32["ms"] / 2, "dtype": "f32",
                            "kernel_ms": {k: round(v["ms"], 3) for k, v in fp32["ktimes"].items()},
                            "roofline": bee_layer_roofline(w, fp32["ktimes"], fp32["local_edges"], per, False, hbm, tf_sus, how),
                            "final_checksum": positions_checksum(fp32["final"]),
                            "note": "same workload through the float32 kernels (1e-5 parity with the float64 oracle)"}
        if not args.no_cpu_baseline and world == 1:
            threads = len(os.sched_getaffinity(0))
            rate, desc = cpu_reference_rate(w, threads, budget_nodes=args.cpu_nodes)
            line["cpu_baseline"] = {"value": rate, "unit": "edge-messages/s", "cores": threads, "kind": "port", "sample": desc}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
