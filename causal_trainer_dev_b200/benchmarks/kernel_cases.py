"""Small, self-terminating single-kernel workloads for profiling and roofline numbers.

    python -m causal_trainer_dev_b200.benchmarks.kernel_cases \
        gemm|dgrad|wgrad|layer_gemms|attn_fwd|attn_bwd|moba [one-document|one-document-128k|coherent]|cut_ce|rmsnorm|adamw|adamw_arena

Each case holds a few hundred MB (more than the 126 MB L2, far less than a GB-scale step),
launches its kernel a handful of times, and prints device-timed milliseconds plus the achieved
fraction of the measured peaks (``MEASURED_PEAKS.json`` beside the repository root when present).
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    return json.loads(p.read_text()) if p.exists() else {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "fallback": True}


def timed(fn, iters: int = 5, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def main() -> None:
    from causal_trainer_dev_b200.ops import attention as A, cross_entropy as CE, elementwise as E, gemm as G

    case = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    pk = peaks()
    torch.manual_seed(0)
    out: dict = {"case": case, "peaks": "measured" if "fallback" not in pk else "fallback"}
    dev = "cuda"
    if case in ("gemm", "wgrad", "dgrad"):
        m, n, k = 8192, 8192, 4096
        if case == "gemm":
            a, b = torch.randn(m, k, device=dev).bfloat16(), torch.randn(n, k, device=dev).bfloat16()
            fn = lambda: G.gemm(a, b)  # noqa: E731
        elif case == "dgrad":
            a, b = torch.randn(m, k, device=dev).bfloat16(), torch.randn(k, n, device=dev).bfloat16()
            fn = lambda: G.gemm(a, b, b_mn=True)  # noqa: E731
        else:
            a, b = torch.randn(k, m, device=dev).bfloat16(), torch.randn(k, n, device=dev).bfloat16()
            fn = lambda: G.gemm(a, b, a_mn=True, b_mn=True)  # noqa: E731
        ms = timed(fn)
        tf = 2.0 * m * n * k / ms / 1e9
        out.update(ms=ms, tflops=tf, fraction_of_measured_bf16_peak=tf / pk["bf16_tflops"])
    elif case == "layer_gemms":
        # the GEMMs of one Llama-3-8B layer at 16384 tokens: forward, dgrad and wgrad (bf16 store and
        # fp32 accumulate through TMA reduce-add) of the four projections
        t, dm, ff, qkv = 16384, 4096, 14336, 6144
        x = torch.randn(t, dm, device=dev).bfloat16()
        res = {}
        for name, n_out, k_in in (("qkv", qkv, dm), ("o", dm, dm), ("gate_up", 2 * ff, dm), ("down", dm, ff)):
            a = torch.randn(t, k_in, device=dev).bfloat16()
            w = torch.randn(n_out, k_in, device=dev).bfloat16()
            dy = torch.randn(t, n_out, device=dev).bfloat16()
            g16 = torch.empty(n_out, k_in, device=dev, dtype=torch.bfloat16)
            g32 = torch.zeros(n_out, k_in, device=dev, dtype=torch.float32)
            fl = 2.0 * t * n_out * k_in / 1e9
            res[name] = {
                "fwd_tflops": fl / timed(lambda: G.gemm(a, w)),
                "dgrad_tflops": fl / timed(lambda: G.gemm(dy, w, b_mn=True)),
                "wgrad_bf16_tflops": fl / timed(lambda: G.gemm(dy, a, a_mn=True, b_mn=True, out=g16)),
                "wgrad_f32_accumulate_tflops": fl / timed(lambda: G.gemm(dy, a, a_mn=True, b_mn=True, out=g32, accumulate=True)),
            }
            res[name] = {k: round(v, 1) for k, v in res[name].items()}
        out.update(res)
    elif case in ("attn_fwd", "attn_bwd"):
        b, s, hq, hkv, d = 2, 4096, 32, 8, 128
        q = torch.randn(b, s, hq, d, device=dev).bfloat16()
        k = torch.randn(b, s, hkv, d, device=dev).bfloat16()
        v = torch.randn(b, s, hkv, d, device=dev).bfloat16()
        meta = A.build_attention_meta(torch.ones(b, s, dtype=torch.int32, device=dev))
        o, lse = A.flash_attention_forward(q, k, v, meta)
        if case == "attn_fwd":
            ms = timed(lambda: A.flash_attention_forward(q, k, v, meta))
            flops = 4.0 * b * hq * s * s * d / 2
        else:
            do = torch.randn_like(o)
            ms = timed(lambda: A.flash_attention_backward(q, k, v, o, do, lse, meta))
            flops = 10.0 * b * hq * s * s * d / 2
        tf = flops / ms / 1e9
        out.update(ms=ms, causal_tflops=tf, fraction_of_measured_bf16_peak=tf / pk["bf16_tflops"])
    elif case == "moba":
        # one 32768-token row packed from 4 documents, MoBA block 4096, top-3 gated blocks + the
        # current block, against dense segment-masked flash attention on the same tensors
        from causal_trainer_dev_b200.ops import moba as M

        b, s, hq, hkv, d, block, top_k = 1, 32768, 32, 8, 128, 4096, 4
        if len(sys.argv) > 2 and sys.argv[2] == "one-document-128k":
            s, hq, hkv = 131072, 8, 2          # a quarter of the heads keeps the case within a few GB
        g = torch.Generator().manual_seed(3)
        lens = torch.randint(4096, 12289, (4,), generator=g).tolist()
        lens[-1] = max(1, s - sum(lens[:-1])) if sum(lens[:-1]) < s else 0
        if len(sys.argv) > 2 and sys.argv[2].startswith("one-document"):
            lens = [s]               # a single document: 8 (32 at 128k) blocks, 4 of them visible per query
        seg = torch.zeros(b, s, dtype=torch.int32)
        pos = 0
        for i, n in enumerate(lens):
            n = min(n, s - pos)
            seg[0, pos:pos + n] = i + 1
            pos += n
        seg = seg.to(dev)
        q = torch.randn(b, s, hq, d, device=dev).bfloat16()
        k = torch.randn(b, s, hkv, d, device=dev).bfloat16()
        v = torch.randn(b, s, hkv, d, device=dev).bfloat16()
        if len(sys.argv) > 2 and sys.argv[2] == "coherent":
            # routing that neighbouring queries agree on (what trained models show): every key
            # block carries its own direction and each group of 1024 queries leans towards three
            # of the earlier blocks
            lens = [s]
            seg = torch.ones(b, s, dtype=torch.int32, device=dev)
            blk = torch.arange(s, device=dev) // block
            k = (k.float() * 0.3)
            k[0, torch.arange(s, device=dev), :, blk] += 6.0
            k = k.bfloat16()
            qf = q.float() * 0.3
            grp = torch.arange(s, device=dev) // 1024
            for j in range(3):
                want = (grp * 7 + j * 3) % torch.clamp(blk, min=1)
                qf[0, torch.arange(s, device=dev), :, want] += 6.0
            q = qf.bfloat16()
        meta = A.build_attention_meta(seg)
        groups = M.build_groups(q, k, meta, block, top_k)
        og, lseg = M.moba_grouped_forward(q, k, v, meta, groups)
        do = torch.randn_like(og)
        od, lsed = A.flash_attention_forward(q, k, v, meta)
        work = groups.work_summary()
        nt = s // 128
        out.update(
            shape=dict(tokens=s, q_heads=hq, kv_heads=hkv, head_dim=d, block=block, top_k=top_k),
            document_lengths=lens, grouped_work=work,
            # a fingerprint of the grouping and of the grouped output (the grouping is a pure function
            # of the routing, so variants of the grouping kernels must reproduce it bit for bit)
            grouping_fingerprint=[int(groups.pos_of.to(torch.int64).sum()), int(groups.row_of.to(torch.int64).sum()),
                                  float(og.double().sum()), float(lseg.double().sum())],
            # 128 x 128 score tiles: grouped history + own-block causal pass, against dense causal attention
            grouped_tiles=work["history_tiles"] + hq * nt * (block // 128 + 1) // 2,
            dense_causal_tiles=hq * nt * (nt + 1) // 2,
            grouping_ms=timed(lambda: M.build_groups(q, k, meta, block, top_k)),
            grouped_fwd_ms=timed(lambda: M.moba_grouped_forward(q, k, v, meta, groups)),
            dense_fwd_ms=timed(lambda: A.flash_attention_forward(q, k, v, meta)),
            grouped_bwd_ms=timed(lambda: M.moba_grouped_backward(q, k, v, og, do, lseg, meta, groups)),
            dense_bwd_ms=timed(lambda: A.flash_attention_backward(q, k, v, od, do, lsed, meta)),
        )
        if s <= 32768:
            # the list-driven variant: one masked flash pass over the union of a tile's selections
            routing = M.build_routing(q, k, meta, block, top_k)
            o, lse = M.moba_forward(q, k, v, meta, routing)
            out.update(
                lists_visited_tile_fraction=routing.visited_fraction,
                lists_routing_ms=timed(lambda: M.build_routing(q, k, meta, block, top_k)),
                lists_fwd_ms=timed(lambda: M.moba_forward(q, k, v, meta, routing)),
                lists_bwd_ms=timed(lambda: M.moba_backward(q, k, v, o, do, lse, meta, routing)),
            )
    elif case == "cut_ce":
        rows, d, vocab = 4096, 4096, 128256
        h = torch.randn(rows, d, device=dev).bfloat16()
        w = (0.02 * torch.randn(vocab, d, device=dev)).bfloat16()
        t = torch.randint(0, vocab, (rows,), device=dev)
        wt = torch.ones(rows, device=dev)
        ms = timed(lambda: CE.cut_ce_forward(h, w, t, wt))
        tf = 2.0 * rows * d * vocab / ms / 1e9
        out.update(ms=ms, tflops=tf, fraction_of_measured_bf16_peak=tf / pk["bf16_tflops"])
    elif case == "rmsnorm":
        rows, d = 32768, 4096
        x = torch.randn(rows, d, device=dev).bfloat16()
        r = torch.randn(rows, d, device=dev).bfloat16()
        w = torch.ones(d, device=dev).bfloat16()
        ms = timed(lambda: E.rmsnorm_forward(x, w, 1e-6, residual=r))
        gbs = 4.0 * rows * d * 2 / ms / 1e6
        out.update(ms=ms, gbs=gbs, fraction_of_measured_copy_bandwidth=gbs / pk["hbm_gbs"])
    elif case == "adamw":
        n = 1 << 27
        p, g, m, v = (torch.randn(n, device=dev).bfloat16() for _ in range(4))
        v.abs_()
        clip = torch.ones(1, device=dev)
        ms = timed(lambda: E.adamw_update(p, g, m, v, lr=1e-4, b1=0.9, b2=0.999, eps=1e-8, decay=0.1, step=2, clip=clip))
        gbs = 7.0 * n * 2 / ms / 1e6
        out.update(ms=ms, gbs=gbs, fraction_of_measured_copy_bandwidth=gbs / pk["hbm_gbs"])
    elif case == "adamw_arena":
        # the sharded runtime's sweep: one launch over a flat arena cut into decay / no-decay regions
        n = 1 << 28
        p, g, m, v = (torch.randn(n, device=dev).bfloat16() for _ in range(4))
        v.abs_()
        clip = torch.ones(1, device=dev)
        cuts = sorted({0, n, *(int(x) // 8 * 8 for x in torch.linspace(0, n, 70).tolist())})
        bounds = torch.tensor(cuts, dtype=torch.int64, device=dev)
        modes = torch.tensor([i % 2 for i in range(len(cuts) - 1)], dtype=torch.int32, device=dev)
        ms = timed(lambda: E.adamw_regions(p, g, m, v, bounds, modes, lr=1e-4, b1=0.9, b2=0.999, eps=1e-8, decay=0.1,
                                           step=2, clip=clip))
        gbs = 7.0 * n * 2 / ms / 1e6
        out.update(ms=ms, gbs=gbs, fraction_of_measured_copy_bandwidth=gbs / pk["hbm_gbs"], elements=n)
    else:
        raise SystemExit(f"unknown case {case}")
    print(json.dumps(out))


if __name__ == "__main__":
    main()
