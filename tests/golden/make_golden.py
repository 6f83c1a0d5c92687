"""Generate the golden vectors in this folder by running the reference's own torch code on CPU.

Run where the reference tree is available (it is not needed to *use* the fixtures):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference /path/to/token-rush

Inputs are regenerated from seeds by `oracle.kv_oracle.seeded_bf16` (CPU generator); each
fixture stores a SHA-256 of the input bits so that a change in the generator is detected.
Outputs are exactly what the reference functions returned: `fused.kv_write_prefill`,
`ops.rmsnorm`, `ops.apply_rope`, `ops.rope_table`, `ops.attn_decode`, `ops.attn_prefill`,
`state.State`, and the masked-SDPA composition the reference's window/ring tests use
(tests/test_fused.py:343-380).  The commit arithmetic is the expression of
tokenrush/model.py:306-311 evaluated with torch.
"""
import argparse
import hashlib
import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import kv_oracle as O  # noqa: E402


def sha(*arrs):
    h = hashlib.sha256()
    for a in arrs:
        h.update(np.ascontiguousarray(a).tobytes())
    return np.frombuffer(h.digest(), dtype=np.uint8)


def bf(bits):
    return O.bits_to_torch_bf16(bits)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference tree (the directory that holds tokenrush/)")
    ap.add_argument("--only", default=None, help="write just this fixture (e.g. add_rmsnorm)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from tokenrush import fused, ops                       # the reference
    from tokenrush.config import ModelConfig
    from tokenrush.state import State

    cfg = ModelConfig(hidden=5120, n_layers=4, layer_types=("linear_attention",) * 3 + ("full_attention",),
                      vocab=1024, ffn=1024, n_heads=24, n_kv_heads=4, head_dim=256, rotary_dim=64,
                      rope_theta=1e7, gdn_k_heads=16, gdn_v_heads=48, gdn_k_dim=128, gdn_v_dim=128, conv_k=4,
                      eps=1e-6, max_pos=4096, eos_ids=(0,))           # tests/test_ops.py:24-27
    HQ, HKV, D = 24, 4, 256
    f8 = torch.float8_e4m3fn

    # ---- 0. residual add + RMSNorm, the torch chain the reference tests its add_rmsnorm kernel
    # against (tests/test_fused.py:21-28,241-246,326-331): ops.rmsnorm / dflash.rmsnorm_plain over x + h
    from tokenrush.dflash import rmsnorm_plain
    xb_, hb_, wb_ = O.seeded_bf16(401, 3, 5120), O.seeded_bf16(402, 3, 5120, std=0.3), O.seeded_bf16(403, 5120, std=0.5)
    x_, h_, w_ = bf(xb_), bf(hb_), bf(wb_)
    parts = torch.Generator().manual_seed(404)
    hp = torch.randn(4, 3, 5120, generator=parts) * 0.2                       # split-K partial rows, fp32
    xs = (x_.float() + hp.sum(0).to(torch.bfloat16).float()).to(torch.bfloat16)
    np.savez_compressed(os.path.join(HERE, "add_rmsnorm.npz"), x_bits=xb_, h_bits=hb_, w_bits=wb_, h_parts=hp.numpy(),
                        xo_bits=O.torch_bf16_to_bits(x_ + h_), y_bits=O.torch_bf16_to_bits(ops.rmsnorm(x_ + h_, w_, 1e-6)),
                        y_noh_bits=O.torch_bf16_to_bits(ops.rmsnorm(x_, w_, 1e-6)),
                        y_plain_bits=O.torch_bf16_to_bits(rmsnorm_plain(x_ + h_, w_ + 1, 1e-6)),
                        xo_parts_bits=O.torch_bf16_to_bits(xs), y_parts_bits=O.torch_bf16_to_bits(ops.rmsnorm(xs, w_, 1e-6)))
    if args.only == "add_rmsnorm":
        return

    # ---- 1. FP8 append: random rows + edge rows ------------------------------------------
    T = 40
    kb = O.seeded_bf16(101, HKV, T, D)
    vb = O.seeded_bf16(102, HKV, T, D)
    k, v = bf(kb).clone(), bf(vb).clone()
    k[0, 0] = 0.0                                            # all-zero row -> floor scale
    k[1, 1] = 1e-8                                           # below the amax floor
    k[2, 2] *= 1000.0                                        # large magnitude
    k[3, 3] = 0.0; k[3, 3, 17] = -3.5                        # one spike, rest zero
    v[0, 4] = -0.0                                           # negative zeros
    v[1, 5] *= 1e-3                                          # small magnitude
    v[2, 6, :] = torch.linspace(-1, 1, D).to(torch.bfloat16)  # quotients through the subnormal range
    v[2, 6, 0] = 448.0
    v[3, 7] = 7.0                                            # constant row: every code 448
    kb, vb = O.torch_bf16_to_bits(k), O.torch_bf16_to_bits(v)
    st = State(cfg, 64, "cpu", kv_dtype=f8)
    fused.kv_write_prefill(k, v, st, 0, 5)
    np.savez_compressed(os.path.join(HERE, "fp8_append.npz"), pos=5, k_bits=kb, v_bits=vb,
                        k_codes=st.k[0].view(torch.uint8).numpy(), v_codes=st.v[0].view(torch.uint8).numpy(),
                        k_scale=st.k_scale[0].numpy(), v_scale=st.v_scale[0].numpy(),
                        bytes_per_token=st.kv_bytes_per_token)

    # ---- 2. decode (M = 1) and M-row verify over an FP8 cache ------------------------------
    L0 = 90
    kb = O.seeded_bf16(201, HKV, L0 + 5, D)
    vb = O.seeded_bf16(202, HKV, L0 + 5, D)
    qb = O.seeded_bf16(203, 5, HQ, D)
    st = State(cfg, 128, "cpu", kv_dtype=f8)
    fused.kv_write_prefill(bf(kb)[:, :L0], bf(vb)[:, :L0], st, 0, 0)
    fused.kv_write_prefill(bf(kb)[:, L0:L0 + 1], bf(vb)[:, L0:L0 + 1], st, 0, L0)     # the decode step's append
    Kd = st.k[0, :, :L0 + 1].float() * st.k_scale[0, :, :L0 + 1, None]                # tests/test_fused.py:299
    Vd = st.v[0, :, :L0 + 1].float() * st.v_scale[0, :, :L0 + 1, None]
    q1 = bf(qb)[:1].transpose(0, 1).float()                                           # [HQ, 1, D]
    o1 = ops.attn_decode(q1, Kd, Vd).transpose(0, 1).contiguous()                     # [1, HQ, D]
    fused.kv_write_prefill(bf(kb)[:, L0:L0 + 5], bf(vb)[:, L0:L0 + 5], st, 0, L0)     # a 5-row verify step
    Kd = st.k[0, :, :L0 + 5].float() * st.k_scale[0, :, :L0 + 5, None]
    Vd = st.v[0, :, :L0 + 5].float() * st.v_scale[0, :, :L0 + 5, None]
    o5 = ops.attn_prefill(bf(qb).transpose(0, 1).float().contiguous(), Kd, Vd, L0).transpose(0, 1).contiguous()
    gate_b = O.seeded_bf16(204, 5, HQ, D)
    gated = (o5.to(torch.bfloat16) * torch.sigmoid(bf(gate_b)))                        # tokenrush/model.py:149
    np.savez_compressed(os.path.join(HERE, "decode_attn.npz"), L0=L0, in_sha=sha(kb, vb, qb, gate_b),
                        out_m1=o1.numpy(), out_m5=o5.numpy(), gated_m5=O.torch_bf16_to_bits(gated))

    # ---- 3. q/k RMSNorm + partial rope (the front half of attn_prep) ------------------------
    M, pos = 3, 1000
    qkvb = O.seeded_bf16(301, M, HQ * 2 * D + 2 * HKV * D)
    qwb = O.seeded_bf16(302, D, std=0.5)
    kwb = O.seeded_bf16(303, D, std=0.5)
    cos, sin = ops.rope_table(2048, cfg.rotary_dim, cfg.rope_theta, "cpu")
    qkv = bf(qkvb)
    kv_dim = HKV * D
    qg, kk, vv = torch.split(qkv, [HQ * 2 * D, kv_dim, kv_dim], dim=-1)               # tokenrush/model.py:123-132
    qg = qg.view(M, HQ, 2 * D)
    qq = ops.rmsnorm(qg[..., :D], bf(qwb), cfg.eps).transpose(0, 1)
    kk = ops.rmsnorm(kk.view(M, HKV, D), bf(kwb), cfg.eps).transpose(0, 1)
    idx = pos + torch.arange(M)
    c, s_ = cos.index_select(0, idx), sin.index_select(0, idx)
    qq = ops.apply_rope(qq, c, s_)
    kk = ops.apply_rope(kk, c, s_)
    sel = np.array([0, 1, 2, 1000, 1001, 1002, 2047])
    np.savez_compressed(os.path.join(HERE, "prep.npz"), M=M, pos=pos, in_sha=sha(qkvb, qwb, kwb),
                        q_bits=O.torch_bf16_to_bits(qq.transpose(0, 1).contiguous()),
                        k_bits=O.torch_bf16_to_bits(kk.contiguous()),
                        table_rows=sel, cos_bits=O.torch_bf16_to_bits(cos[sel]), sin_bits=O.torch_bf16_to_bits(sin[sel]))

    # ---- 4. window + ring + block keys (DFlash draft attention), bf16 cache ------------------
    hq, hkv, d, B, W = 32, 8, 128, 8, 48
    R = 64                                                    # ring_size(48, 8) == 64
    pos = 150
    kfb = O.seeded_bf16(401, hkv, pos, d); vfb = O.seeded_bf16(402, hkv, pos, d)
    qb = O.seeded_bf16(403, B, hq, d)
    kbb = O.seeded_bf16(404, hkv, B, d); vbb = O.seeded_bf16(405, hkv, B, d)
    Kfull, Vfull = bf(kfb), bf(vfb)
    lo = pos - (W - 1)
    keys = torch.arange(lo, pos); blk = pos + torch.arange(B)
    mask = torch.cat([(blk[:, None] - keys[None, :]) < W, torch.ones(B, B, dtype=torch.bool)], 1)
    Kf = torch.cat([Kfull[:, lo:pos], bf(kbb)], 1).float(); Vf = torch.cat([Vfull[:, lo:pos], bf(vbb)], 1).float()
    ref = F.scaled_dot_product_attention(bf(qb).transpose(0, 1).float()[None], Kf[None], Vf[None], attn_mask=mask,
                                         enable_gqa=True)[0].transpose(0, 1).contiguous()
    np.savez_compressed(os.path.join(HERE, "window_block.npz"), pos=pos, window=W, ring=R, B=B,
                        in_sha=sha(kfb, vfb, qb, kbb, vbb), out=ref.numpy())

    # ---- 5. chunked prefill over an FP8 cache, chunk starts mid-cache ------------------------
    pos, T = 37, 50
    kb = O.seeded_bf16(501, HKV, pos + T, D); vb = O.seeded_bf16(502, HKV, pos + T, D)
    qb = O.seeded_bf16(503, T, HQ, D)
    st = State(cfg, 128, "cpu", kv_dtype=f8)
    fused.kv_write_prefill(bf(kb)[:, :pos], bf(vb)[:, :pos], st, 0, 0)
    fused.kv_write_prefill(bf(kb)[:, pos:], bf(vb)[:, pos:], st, 0, pos)
    Kd = st.k[0, :, :pos + T].float() * st.k_scale[0, :, :pos + T, None]
    Vd = st.v[0, :, :pos + T].float() * st.v_scale[0, :, :pos + T, None]
    o = ops.attn_prefill(bf(qb).transpose(0, 1).float().contiguous(), Kd, Vd, pos).transpose(0, 1).contiguous()
    rows = np.array([0, 1, 7, 24, 31, 32, 49])               # a sample of query rows keeps the fixture small
    np.savez_compressed(os.path.join(HERE, "prefill.npz"), pos=pos, T=T, in_sha=sha(kb, vb, qb), rows=rows,
                        out=o.numpy()[rows])

    # ---- 6. speculative commit ------------------------------------------------------------
    g = torch.Generator().manual_seed(601)
    cases = []
    for _ in range(64):
        K = int(torch.randint(1, 8, (1,), generator=g))
        pred = torch.randint(0, 4, (K + 1,), generator=g)
        drafts = torch.randint(0, 4, (K,), generator=g)
        keep = int(torch.randint(0, K + 1, (1,), generator=g))
        drafts[:keep] = pred[:keep]                           # plant an accepted prefix
        pos0 = int(torch.randint(0, 100000, (1,), generator=g))
        match = (pred[:K] == drafts).long()                   # tokenrush/model.py:306-311
        n = match.cumprod(0).sum().view(1)
        tok = pred.gather(0, n)
        row = np.full(20, -1, dtype=np.int64)
        row[0], row[1], row[2], row[3], row[4] = K, pos0, int(n), int(tok), pos0 + int(n) + 1
        row[5:5 + K + 1] = pred.numpy(); row[13:13 + K] = drafts.numpy()
        cases.append(row)
    np.savez_compressed(os.path.join(HERE, "commit.npz"), cases=np.stack(cases))
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    main()
