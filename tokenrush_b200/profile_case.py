"""Small, self-ending cases for profiling one kernel of the library under ncu.

    python -m tokenrush_b200.profile_case decode  [--rows 131072] [--m 1] [--layers 2] [--iters 3]
    python -m tokenrush_b200.profile_case prefill [--rows 16384] [--t 2048]

The cache is filled with random e4m3 codes and plausible scales (no quantisation pass, so few
launches precede the kernel of interest); inputs exceed L2 for the decode case, and everything
stays within a few GB.
"""
import argparse

import torch

import tokenrush_b200 as tb

HQ, HKV, D = 24, 4, 256


def random_fill_(state):
    for t in (state.k, state.v):
        codes = torch.randint(0, 0x7E, t.shape, device="cuda", dtype=torch.uint8)
        sign = torch.randint(0, 2, t.shape, device="cuda", dtype=torch.uint8) << 7
        t.view(torch.uint8).copy_(codes | sign)
    state.k_scale.uniform_(0.006, 0.011)
    state.v_scale.uniform_(0.006, 0.011)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["decode", "prefill"])
    ap.add_argument("--rows", type=int, default=None)
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--t", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    f8 = torch.float8_e4m3fn
    if a.kernel == "decode":
        rows = a.rows or 131072
        cfg = tb.AttnConfig(n_attn=a.layers)
        st = tb.State(cfg, rows + 64, "cuda", kv_dtype=f8)
        random_fill_(st)
        st.set_pos(rows - a.m)
        q = torch.randn(a.m, HQ * D, device="cuda").to(torch.bfloat16)
        for _ in range(a.iters):
            for l in range(a.layers):
                tb.fused.attn_decode_fused(q, None, st.k[l], st.v[l], st.pos_t, cfg, st.k_scale[l], st.v_scale[l])
    else:
        rows = a.rows or 16384
        cfg = tb.AttnConfig(n_attn=1)
        st = tb.State(cfg, rows + a.t + 64, "cuda", kv_dtype=f8)
        random_fill_(st)
        q = torch.randn(a.t, HQ, D, device="cuda").to(torch.bfloat16)
        for _ in range(min(a.iters, 2)):
            tb.fused.attn_prefill_fused(q, st.k[0], st.v[0], rows, cfg, st.k_scale[0], st.v_scale[0])
    torch.cuda.synchronize()
    print("ok, device status", tb._lib.device_status())


if __name__ == "__main__":
    main()
