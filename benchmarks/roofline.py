"""Roofline bounds of the fused compute + collective paths.

For every named path: t_flop (FLOPs over the measured bf16 GEMM throughput), t_hbm (weight
bytes over the measured copy bandwidth) and t_link (bytes that must cross NVLink per GPU over
the measured peer-copy rate), and the bound = the largest of the three.  The denominators
come from MEASURED_PEAKS.json next to the repository root when present, else from the
fallback figures of an earlier measurement on the same pool.

  python benchmarks/roofline.py [--tp 8] [--measured path.json]

``--measured`` takes the JSON printed by benchmarks/kernels/bench_fused_tp.py and adds the
achieved fraction (bound / measured time) for the shapes it contains.
"""
import argparse
import json
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LINK_GBS = 770.0          # measured peer copy, per direction per GPU (nominal 900)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["bf16_tflops"], d["bf16_tflops_sustained"], d["hbm_gbs"], "measured"
    return 1590.0, 1400.0, 6650.0, "fallback"


def allreduce_bytes(payload: float, p: int, mode: str) -> float:
    """Bytes one GPU sends for an all-reduce of ``payload`` bytes."""
    if mode == "oneshot":
        return (p - 1) * payload
    if mode == "twoshot":
        return 2.0 * (p - 1) / p * payload
    if mode == "reduce_scatter" or mode == "all_gather":
        return (p - 1) / p * payload
    raise ValueError(mode)


def row(name, M, N, K, p, coll, payload, burst, hbm):
    flop = 2.0 * M * N * K
    t_flop = flop / (burst * 1e12)
    t_hbm = N * K * 2.0 / (hbm * 1e9)
    t_link = allreduce_bytes(payload, p, coll) / (LINK_GBS * 1e9) if p > 1 else 0.0
    bound = max(t_flop, t_hbm, t_link)
    which = {t_flop: "tensor", t_hbm: "HBM", t_link: "link"}[bound]
    return dict(path=name, M=M, N=N, K=K, collective=coll, t_flop_us=t_flop * 1e6,
                t_hbm_us=t_hbm * 1e6, t_link_us=t_link * 1e6, bound_us=bound * 1e6, bound=which)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--measured", default=None)
    a = ap.parse_args()
    burst, sustained, hbm, src = peaks()
    p = a.tp
    H, I, V = 4096, 14336, 128256                       # Llama-3-8B
    rows = []
    for T in (256, 8192):
        s = T * H * 2.0
        mode = "oneshot" if (T <= 1024 or p == 2) else "twoshot"
        rows.append(row(f"o_proj -> all-reduce, T={T}", T, H, H // p, p, mode, s, burst, hbm))
        rows.append(row(f"down_proj -> all-reduce, T={T}", T, H, I // p, p, mode, s, burst, hbm))
        rows.append(row(f"all-gather -> qkv_proj (SP), T={T}", T, 6144 // p, H, p, "all_gather",
                        s, burst, hbm))
    rows.append(row("LM head -> logits all-gather, B=256", 256, V // p, H, p, "all_gather",
                    256 * V * 2.0, burst, hbm))
    # expert-parallel dispatch / combine (DeepSeek-V3 shapes, 128 tokens per rank, k = 8)
    for name, rows_per_rank, width in (("EP dispatch (bf16 rows + ids + weights)", 128 * 8,
                                        7168 * 2 + 64),
                                       ("EP dispatch (fp8 rows + group scales + ids + weights)",
                                        128 * 8, 7168 + 7168 // 128 * 4 + 64),
                                       ("EP combine (bf16 rows)", 128 * 8, 7168 * 2)):
        b = rows_per_rank * width * (p - 1) / p
        t = b / (LINK_GBS * 1e9)
        rows.append(dict(path=name, collective="all_to_all", t_flop_us=0.0, t_hbm_us=0.0,
                         t_link_us=t * 1e6, bound_us=t * 1e6, bound="link"))
    measured = {}
    if a.measured:
        d = json.load(open(a.measured))
        for r in d.get("results", []):
            measured[(r["M"], r["K"])] = r
    print(f"peaks ({src}): bf16 burst {burst:.0f} TFLOP/s, sustained {sustained:.0f}, "
          f"HBM {hbm:.0f} GB/s, link {LINK_GBS:.0f} GB/s per direction; tp = {p}")
    print(f"{'path':44s} {'t_flop':>8s} {'t_hbm':>8s} {'t_link':>8s} {'bound':>8s}  limit")
    for r in rows:
        line = (f"{r['path']:44s} {r['t_flop_us']:8.1f} {r['t_hbm_us']:8.1f} "
                f"{r['t_link_us']:8.1f} {r['bound_us']:8.1f}  {r['bound']}")
        m = measured.get((r.get("M"), r.get("K")))
        if m:
            best = min(v for k, v in m.items() if k.endswith("shot_us"))
            line += f"   measured {best:.1f} us -> {r['bound_us'] / best:.2f} of bound"
        print(line)


if __name__ == "__main__":
    main()
