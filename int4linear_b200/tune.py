"""Time the tile configurations of the tensor-memory GEMM on given shapes.

    python -m int4linear_b200.tune 1024x1024x1024 512x4096x4096 ...

For every shape, each forced configuration (CTA pairs, and single-CTA tiles 256, 128 and 64
columns wide) and the dispatcher's own choice are timed as a CUDA graph of `--launches` launches
over rotating operand sets that together exceed L2, so the figures carry neither launch overhead
nor a warm L2.  The relative tile times this prints are what the cost model of the dispatcher
(launch_tcgen05 in csrc/gemm_tcgen05.cu) is fitted to.
"""
from __future__ import annotations

import argparse

DEFAULT_SHAPES = ["1024x1024x1024", "2048x2048x2048", "2048x2048x1024", "512x4096x4096", "256x8192x4096",
                  "1024x4096x1024", "128x14336x4096", "64x14336x4096", "4096x4096x4096", "4096x1024x4096",
                  "3072x3072x3072", "1536x6144x2048", "8192x1024x1024"]
CONFIGS = {"auto": (0, -1), "pairs": (0, 1), "c256": (256, 0), "c128": (128, 0), "c64": (64, 0)}
L2_BYTES = 126e6


def time_shape(m: int, n: int, k: int, launches: int, device) -> dict[str, float]:
    """Microseconds per launch for every configuration."""
    import torch
    from . import linear, set_tuning, uniform_s4_packed
    ws = m * k // 2 + n * k // 2 + 4 * m * n
    sets = min(64, int(2 * L2_BYTES // ws) + 1)
    xs = [torch.from_numpy(uniform_s4_packed(1, m, k)).to(device)]
    ws_ = [torch.from_numpy(uniform_s4_packed(2, n, k)).to(device)]
    xs += [xs[0].clone() for _ in range(sets - 1)]
    ws_ += [ws_[0].clone() for _ in range(sets - 1)]
    ys = [torch.empty((m, n), dtype=torch.int32, device=device) for _ in range(sets)]
    out = {}
    try:
        for name, (tile, pairs) in CONFIGS.items():
            if name == "pairs" and m <= 128:
                continue  # a lone row block would leave the second CTA of a pair idle
            set_tuning(tile, False, pairs)
            linear(xs[0], ws_[0], out=ys[0])  # the library's first call must not happen inside a capture
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for i in range(launches):
                        linear(xs[i % sets], ws_[i % sets], out=ys[i % sets])
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            out[name] = a.elapsed_time(b) / launches * 1e3
    finally:
        set_tuning(0, False, -1)
    return out


def main(argv=None) -> None:
    import torch
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("shapes", nargs="*", default=DEFAULT_SHAPES, help="MxNxK")
    ap.add_argument("--launches", type=int, default=40)
    args = ap.parse_args(argv)
    device = torch.device("cuda", 0)
    for shape in args.shapes:
        m, n, k = (int(v) for v in shape.lower().split("x"))
        t = time_shape(m, n, k, args.launches, device)
        best = min((v, name) for name, v in t.items() if name != "auto")
        cols = "  ".join(f"{name}={v:.1f}" for name, v in t.items())
        print(f"{m}x{n}x{k}: {cols}   best={best[1]}  auto/best={t['auto'] / best[0]:.2f}")


if __name__ == "__main__":
    main()
