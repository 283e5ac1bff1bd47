"""Cycle counts per phase of the two fused tensor-core edge kernels (diagnostics).

    python -m ld_b200.phase_profile painn     # ld_painn_message_bf16_tc, 4 periodic boxes x 2048, n = 128
    python -m ld_b200.phase_profile bee       # ld_bee_messages_scalar_bf16_tc, 128 polymers x 256, (128, 64, 32, 128)

The kernels have a second instance with clock64() laps around their phases; it is selected while a
counter buffer is registered with ld_debug_set_phase_counters. The numbers are cycles summed over
blocks (thread 0 of each block), printed per 128-edge tile; the instrumented instance spills a few
registers, so the production kernel is slightly faster than the sum shown."""
import sys

import torch

from . import _lib, graph_layers as GL

PAINN_LABELS = ["geometry", "radial features", "wait layer 1 MMAs", "epilogue 1", "wait layer 2 MMAs", "epilogue 2",
                "wait layer 3 MMAs", "per-node sums: join + barrier", "gather + message staging", "MMA lane: waiting for weights",
                "producer: waiting for a free stage", "per-node sums: row halves"]
BEE_LABELS = ["geometry", "products (gather)", "wait Y MMAs", "epilogue Y", "wait layer 1 MMAs", "epilogue 1",
              "wait layer 2 MMAs", "epilogue 2", "wait layer 3 MMAs", "staging", "per-node sums"]


def _run(fn, labels, worker_slots):
    buf = torch.zeros(16, dtype=torch.int64, device="cuda")
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.no_grad():
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        plain_ms = e0.elapsed_time(e1)
        _lib.lib().ld_debug_set_phase_counters(buf.data_ptr())
        try:
            fn()
            torch.cuda.synchronize()
        finally:
            _lib.lib().ld_debug_set_phase_counters(None)
    return buf.cpu().tolist(), plain_ms


def painn():
    from . import painn as P
    torch.manual_seed(0)
    n, B, N, r0, box = 128, 4, 2048, 4.0, (12.6,) * 3
    msg = P.Message(r0, n, 8, "gaussian").cuda()
    msg.precision = "bf16"
    pos = torch.rand(B, N, 3, device="cuda") * 12.6
    x_a, x_v = torch.randn(B, N, n, device="cuda"), torch.randn(B, N, n, 3, device="cuda")
    with torch.no_grad():
        graph = GL.Graph.radius_graph(r0, box, pos)
    vals, ms = _run(lambda: msg(graph, x_a, x_v, graph.rij), PAINN_LABELS, 9)
    return graph.src.numel(), vals, ms, PAINN_LABELS, (0, 1, 2, 3, 4, 5, 6, 7, 8, 11)


def bee():
    from . import bee as Bm
    torch.manual_seed(0)
    B, N, r0 = 128, 256, 5.0
    mes = Bm.set_precision(Bm.Messages(r0, 128, 64, 32, 128).cuda(), "bf16")
    g = torch.Generator().manual_seed(1)
    pos = torch.cumsum(torch.randn(B, N, 3, generator=g) / 3 ** 0.5, dim=1).cuda()
    x_a = torch.randn(B, N, 128, device="cuda")
    x_v = torch.randn(B, N, 64, 3, device="cuda")
    x_d = torch.randn(B, N, 32, 3, 3, device="cuda")
    with torch.no_grad():
        graph = GL.Graph.radius_graph(r0, None, pos)
    vals, ms = _run(lambda: mes(graph, graph.rij, x_a, x_v, x_d), BEE_LABELS, 11)
    return graph.src.numel(), vals, ms, BEE_LABELS, tuple(range(11))


def main(argv):
    which = argv[1] if len(argv) > 1 else "painn"
    E, vals, ms, labels, nworker = (painn if which == "painn" else bee)()
    tiles = E / 128
    print(f"{which}: E = {E} edges, {tiles:.0f} tiles of 128 edges, layer forward {ms:.3f} ms (production instance); cycles per tile:")
    for i, lab in enumerate(labels):
        print(f"  {lab:36s} {vals[i] / tiles:9.0f}")
    total_label = "sum over the working warps' phases"
    print(f"  {total_label:36s} {sum(vals[i] for i in nworker) / tiles:9.0f}")


if __name__ == "__main__":
    main(sys.argv)
