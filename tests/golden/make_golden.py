"""Generate golden vectors by running the UNMODIFIED reference on seeded inputs.

Usage (only where a checkout of the reference project exists):
    python tests/golden/make_golden.py /path/to/DiRotQ

Writes tests/golden/*.npz.  bf16 tensors are stored as their uint16 bit patterns
(key suffix ``__bf16``) so the files stay exact and numpy-only.
"""
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))


def to_np(d):
    out = {}
    for k, v in d.items():
        if v is None:
            continue
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().contiguous()
            if v.dtype == torch.bfloat16:
                out[k + "__bf16"] = v.view(torch.int16).numpy().view(np.uint16)
            elif v.dtype == torch.float16:
                out[k + "__f16"] = v.view(torch.int16).numpy().view(np.uint16)
            else:
                out[k] = v.numpy()
        else:
            out[k] = np.asarray(v)
    return out


def main(ref_root):
    sys.path.insert(0, ref_root)
    import dirotq_fused_unrotation as slow
    import dirotq_fused_unrotation_fast as fast
    from utils import quant_utils as qu
    from utils.hadamard_utils import random_orthogonal_matrix

    def orth(n, seed):
        torch.manual_seed(seed)
        return random_orthogonal_matrix(n, device="cpu").float()

    def acts(B, T, D, seed, heavy=True):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(B, T, D, generator=g)
        if heavy:
            v = torch.linalg.qr(torch.randn(D, 8, generator=g))[0]
            x = x + (torch.randn(B, T, 8, generator=g) * 4.4) @ v.T
            x[..., 3] = x[..., 3] * 9.0
        return x.to(torch.bfloat16)

    def build(D, N, seed, *, rotation=None, rph=None, H=None, d=None, cfg=None, weight_mode="int", w_groupsize=None):
        torch.manual_seed(seed)
        lin = nn.Linear(D, N, bias=True).to(torch.bfloat16)
        w = qu.ActQuantWrapper(lin)
        w.quantizer.configure(**cfg)
        if rotation is not None:
            w.rotation = rotation
        if rph is not None:
            w.rotation_per_head = rph
            w.num_heads, w.head_dim = H, d
        holder = nn.ModuleDict({"l": w})
        wg = cfg["groupsize"] if w_groupsize is None else w_groupsize
        if weight_mode == "int":
            qu.rtn_quantize_weights(holder, bits=4, groupsize=wg, sym=True)
        else:
            qu.nvfp4_rtn_quantize_weights(holder, groupsize=wg)
        assert w._unrot_fused
        return w

    def run_case(name, w, x):
        out = {"x": x, "weight": w.module.weight.data, "bias": w.module.bias.data}
        if w.rotation is not None:
            out["rotation"] = w.rotation
        if w.rotation_per_head is not None:
            out["rotation_per_head"] = w.rotation_per_head
        q = w.quantizer
        out["cfg"] = np.array([q.bits, q.groupsize, int(q.sym), q.high_bits_length,
                               1 if q.quant_dtype == "nvfp4" else 0], dtype=np.int64)
        # fast (bf16) path: the bit contract
        rot_saved, rph_saved = w.rotation, w.rotation_per_head
        if rot_saved is not None:
            w.rotation = rot_saved.to(torch.bfloat16)
        if rph_saved is not None:
            w.rotation_per_head = rph_saved.to(torch.bfloat16)
        with torch.no_grad():
            out["y_fast"] = fast._fused_forward_fast(w, x)
            # intermediate tensors of the fast path, recomputed with the same calls
            if w.rotation is not None:
                x_rot = (x.reshape(-1, x.shape[-1]) @ w.rotation).reshape(x.shape)
                q.find_params(x_rot)
                out["x_rot_fast"] = x_rot
                out["xq_fast"] = q(x_rot)
                if q.scale is not None and q.scale.numel() > 1:
                    out["scale_fast"] = q.scale
                    out["zero_fast"] = q.zero
            elif w.rotation_per_head is not None:
                H, d = w.num_heads, w.head_dim
                hlen = q.high_bits_length
                d_q = d - hlen
                xh = x.reshape(*x.shape[:-1], H, d)
                xr = torch.einsum('...hd,hde->...he', xh, w.rotation_per_head)
                xre = torch.cat([xr[..., :d_q].reshape(*x.shape[:-1], H * d_q),
                                 xr[..., d_q:].reshape(*x.shape[:-1], H * hlen)], dim=-1)
                sh, sg = q.high_bits_length, q.groupsize
                q.high_bits_length, q.groupsize = H * hlen, d_q
                q.find_params(xre)
                out["x_rot_fast"] = xre
                out["xq_fast"] = q(xre)
                if q.scale is not None and q.scale.numel() > 1:
                    out["scale_fast"] = q.scale
                    out["zero_fast"] = q.zero
                q.high_bits_length, q.groupsize = sh, sg
        w.rotation, w.rotation_per_head = rot_saved, rph_saved
        with torch.no_grad():
            out["y_slow"] = slow._fused_forward(w, x)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **to_np(out))
        print("wrote", name, {k: tuple(v.shape) for k, v in out.items() if hasattr(v, "shape")})

    # GOLDEN_ONLY=hadamard | pertoken: add those fixtures without rewriting the others
    only = os.environ.get("GOLDEN_ONLY")
    _run_case, build_saved = run_case, build
    if only:
        run_case = lambda *a, **k: None
        build = lambda *a, **k: None
    # 1. hidden rotation, INT4 symmetric g64, k=64 passthrough
    D, N = 192, 96
    cfg = dict(bits=4, groupsize=64, sym=True, high_bits_length=64, quant_dtype="int")
    run_case("hidden_int4_sym", build(D, N, 1, rotation=orth(D, 11), cfg=cfg), acts(2, 24, D, 21))
    # 2. the adapters' default: asymmetric INT4
    cfg = dict(bits=4, groupsize=64, sym=False, high_bits_length=64, quant_dtype="int")
    run_case("hidden_int4_asym", build(D, N, 2, rotation=orth(D, 12), cfg=cfg), acts(2, 24, D, 22))
    # 3. q_len % groupsize != 0 (zero padding) and no passthrough tail
    D = 160
    cfg = dict(bits=4, groupsize=64, sym=True, high_bits_length=0, quant_dtype="int")
    run_case("hidden_int4_pad_notail", build(D, N, 3, rotation=orth(D, 13), cfg=cfg), acts(2, 16, D, 23))
    # 4. W4A8 asymmetric
    D = 192
    cfg = dict(bits=8, groupsize=64, sym=False, high_bits_length=64, quant_dtype="int")
    run_case("hidden_int8_asym", build(D, N, 4, rotation=orth(D, 14), cfg=cfg), acts(2, 16, D, 24))
    # 5. NVFP4 g16
    cfg = dict(bits=4, groupsize=16, sym=True, high_bits_length=48, quant_dtype="nvfp4")
    run_case("hidden_nvfp4", build(D, N, 5, rotation=orth(D, 15), cfg=cfg, weight_mode="nvfp4"),
             acts(2, 24, D, 25))
    # 6. per-head rotation (PixArt to_out shape family: d=72, hlen=9 -> groups of 63)
    H, d = 4, 72
    torch.manual_seed(16)
    rph = torch.stack([random_orthogonal_matrix(d, device="cpu").float() for _ in range(H)])
    cfg = dict(bits=4, groupsize=64, sym=True, high_bits_length=9, quant_dtype="int")
    run_case("perhead_int4_sym", build(H * d, N, 6, rph=rph, H=H, d=d, cfg=cfg), acts(2, 16, H * d, 26))
    cfg = dict(bits=4, groupsize=64, sym=False, high_bits_length=9, quant_dtype="int")
    run_case("perhead_int4_asym", build(H * d, N, 7, rph=rph, H=H, d=d, cfg=cfg), acts(2, 16, H * d, 27))
    # SANA family: d=32, hlen=4 -> groups of 28
    H, d = 6, 32
    torch.manual_seed(17)
    rph = torch.stack([random_orthogonal_matrix(d, device="cpu").float() for _ in range(H)])
    cfg = dict(bits=4, groupsize=64, sym=True, high_bits_length=4, quant_dtype="int")
    run_case("perhead_d32_int4_sym", build(H * d, N, 8, rph=rph, H=H, d=d, cfg=cfg), acts(2, 16, H * d, 28))

    # Hadamard layers (use_hadamard: FWHT over the first low_dim channels with sign flips, the rest untouched)
    from utils.hadamard_utils import generate_sign_flips, fast_hadamard_transform
    for name, D, low_dim, hl, seed in (("hadamard_int4_sym", 320, 256, 64, 9), ("hadamard_int4_sym_n128", 192, 128, 64, 10)):
        if only not in (None, "hadamard"):
            break
        cfg = dict(bits=4, groupsize=64, sym=True, high_bits_length=hl, quant_dtype="int")
        torch.manual_seed(seed)
        lin = nn.Linear(D, N, bias=True).to(torch.bfloat16)
        w = qu.ActQuantWrapper(lin)
        w.quantizer.configure(**cfg)
        w.use_hadamard, w.hadamard_low_dim = True, low_dim
        w.hadamard_sign_flips = generate_sign_flips(low_dim, seed=42 + seed)
        holder = nn.ModuleDict({"l": w})
        qu.rtn_quantize_weights(holder, bits=4, groupsize=64, sym=True)
        assert w._unrot_fused
        x = acts(2, 24, D, 30 + seed)
        out = {"x": x, "weight": w.module.weight.data, "bias": w.module.bias.data,
               "sign_flips": w.hadamard_sign_flips, "low_dim": np.array([low_dim], dtype=np.int64),
               "cfg": np.array([4, 64, 1, hl, 0], dtype=np.int64)}
        flips_saved = w.hadamard_sign_flips
        with torch.no_grad():
            w.hadamard_sign_flips = flips_saved.to(torch.bfloat16)
            out["y_fast"] = fast._fused_forward_fast(w, x)
            x_low = x[..., :low_dim] * w.hadamard_sign_flips
            x_rot = torch.cat([fast_hadamard_transform(x_low.float()).to(x.dtype), x[..., low_dim:]], dim=-1)
            w.quantizer.find_params(x_rot)
            out["x_rot_fast"] = x_rot
            out["xq_fast"] = w.quantizer(x_rot)
            out["scale_fast"] = w.quantizer.scale
            w.hadamard_sign_flips = flips_saved.float()
            out["y_slow"] = slow._fused_forward(w, x)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **to_np(out))
        print("wrote", name, {k: tuple(v.shape) for k, v in out.items() if hasattr(v, "shape")})
    if only in (None, "pertoken"):
        # per-token activation scales (groupsize <= 0: ActQuantizer._find_params), weights in groups of 64; q_len = 128
        # and (no tail) q_len = 160, whose last 64-chunk is half padding
        for name, D, hl, sym, seed in (("hidden_int4_sym_pertoken", 192, 64, True, 18), ("hidden_int4_asym_pertoken", 192, 64, False, 19),
                                       ("hidden_int4_asym_pertoken_pad", 160, 0, False, 20)):
            cfg = dict(bits=4, groupsize=-1, sym=sym, high_bits_length=hl, quant_dtype="int")
            _run_case(name, build_saved(D, N, seed, rotation=orth(D, 40 + seed), cfg=cfg, w_groupsize=64), acts(2, 24, D, 50 + seed))
        # per-head rotation with NVFP4 activations (FLUX to_out family: 16 of d channels per head in 16 bits);
        # the reference quantises each head's d - 16 coefficients as one E2M1 group with an unrounded scale
        H, d = 4, 64
        torch.manual_seed(21)
        rph = torch.stack([random_orthogonal_matrix(d, device="cpu").float() for _ in range(H)])
        cfg = dict(bits=4, groupsize=16, sym=True, high_bits_length=16, quant_dtype="nvfp4")
        _run_case("perhead_nvfp4", build_saved(H * d, N, 22, rph=rph, H=H, d=d, cfg=cfg, weight_mode="nvfp4"),
                  acts(2, 24, H * d, 62))
    if only:
        return

    # 7. quantiser-only adversarial inputs (already "rotated"): exact .5 ties after the
    #    bf16 quotient rounding, an all-zero group, a tiny group, negative-only group.
    q = qu.ActQuantizer()
    g = torch.Generator().manual_seed(31)
    xr = torch.randn(1, 64, 256, generator=g)
    xr[0, :, 0] = 7.0                      # scale = 1 -> half-integers are exact ties
    xr[0, :, 1:64] = (torch.randint(-15, 16, (64, 63), generator=g).float() / 2.0)
    xr[0, 3, 64:128] = 0.0                 # all-zero group (scale := 1 rule)
    xr[0, 4, 64:128] = 1e-7 * torch.randn(64, generator=g)   # tiny group
    xr[0, 5, 128:192] = -xr[0, 5, 128:192].abs()              # all-negative group
    xr = xr.to(torch.bfloat16)
    out = {"x_rot": xr}
    for tag, kw in [("int4_sym", dict(bits=4, groupsize=64, sym=True, high_bits_length=64)),
                    ("int4_asym", dict(bits=4, groupsize=64, sym=False, high_bits_length=64)),
                    ("int8_asym", dict(bits=8, groupsize=64, sym=False, high_bits_length=64)),
                    ("int4_sym_f32", dict(bits=4, groupsize=64, sym=True, high_bits_length=64))]:
        q.configure(quant_dtype="int", **kw)
        xin = xr.float() if tag.endswith("f32") else xr
        q.find_params(xin)
        out["xq_" + tag] = q(xin)
        out["scale_" + tag] = q.scale
        out["zero_" + tag] = q.zero
    # NVFP4 ties: normalised values exactly on codebook midpoints
    xn = torch.randn(1, 32, 64, generator=g)
    mids = torch.tensor([-5, -3.5, -2.5, -1.75, -1.25, -0.75, -0.25, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    for t in range(32):
        xn[0, t, 0] = 6.0                  # scale = 1
        xn[0, t, 1:15] = mids
        xn[0, t, 15] = 0.0
    xn[0, 7, 16:32] = 0.0                  # all-zero group -> clamp(1e-5)
    xn[0, 8, 16:32] = 1e-7
    xn = xn.to(torch.bfloat16)
    q.configure(bits=4, groupsize=16, high_bits_length=16, quant_dtype="nvfp4")
    q.find_params(xn)
    out["x_rot_nvfp4"] = xn
    out["xq_nvfp4"] = q(xn)
    np.savez_compressed(os.path.join(HERE, "quantizer_edge.npz"), **to_np(out))
    print("wrote quantizer_edge")

    # 8. weight side
    g = torch.Generator().manual_seed(41)
    W = torch.randn(48, 192, generator=g) * 0.05
    W[5, 64:128] = 0.0
    out = {"W": W,
           "wq_int4_g64": qu._quant_group_int(W.clone(), 4, 64, True),
           "wq_int4_g63": qu._quant_group_int(W[:, :189].clone(), 4, 63, True),
           "wq_nvfp4_g16": qu._quant_group_nvfp4(W.clone(), 16)}
    try:
        sys.path.insert(0, os.path.join(ref_root, "speedup"))
        import nunchaku_pack as npk
        xt = torch.tensor([0.25, -0.25, 0.75, 2.5, -2.5, 5.0, -5.0, 0.1, -0.1, 7.0, -7.0, 1.25])
        out["fp_quantize_in"] = xt
        out["fp_quantize_idx"] = npk.fp_quantize(xt)
        d = npk.convert_dirotq_low_weight_to_nunchaku(W.to(torch.bfloat16)[:, :128].repeat(3, 1)[:128].contiguous()
                                                      .repeat(1, 2), group_size=64)
        out["nunchaku_qweight_shape"] = np.array(d["qweight"].shape)
        out["nunchaku_wscales_shape"] = np.array(d["wscales"].shape)
    except Exception as e:  # pragma: no cover
        print("nunchaku_pack vectors skipped:", e)
    try:
        import weight_only_nvfp4 as wo
        codes, micro, gscale = wo._quantize_nvfp4(W)
        out["wo_codes"] = codes
        out["wo_micro_u8"] = micro.view(torch.uint8)
        out["wo_gscale"] = gscale
    except Exception as e:  # pragma: no cover
        print("weight_only_nvfp4 vectors skipped:", e)
    np.savez_compressed(os.path.join(HERE, "weights.npz"), **to_np(out))
    print("wrote weights")

    # 9. the two-level NVFP4 weight recipe on a wide dynamic range: group magnitudes spread over 2^-16 .. 1 inside a
    #    row (micro-scales down to subnormal and zero), an all-zero row, all-zero and denormal-small groups, and one
    #    group whose effective scale is exactly 1 with every codebook midpoint of both signs in it (tie rule)
    try:
        import weight_only_nvfp4 as wo
        g = torch.Generator().manual_seed(43)
        W2 = torch.randn(64, 512, generator=g)
        W2 = W2 * torch.exp2(torch.randint(-16, 1, (64, 32, 1), generator=g).float()).expand(64, 32, 16).reshape(64, 512)
        W2[3] = 0
        W2[4, :16] = 0
        W2[5, 16:32] = 1e-30
        W2[6, :16] = torch.tensor([6., 0.25, -0.25, 0.75, -0.75, 1.25, -1.25, 1.75, -1.75, 2.5, -2.5, 3.5, -3.5, 5., -5., 0.])
        W2[6, 16:] = W2[6, 16:].clamp(-6, 6)
        codes, micro, gscale = wo._quantize_nvfp4(W2)
        lin = wo.WeightOnlyNVFP4Linear(512, 64, bias=False, device="cpu")
        lin.codes.copy_(codes)
        lin.micro.copy_(micro)
        lin.gscale.copy_(gscale)
        out = {"W": W2, "wo_codes": codes, "wo_micro_u8": micro.view(torch.uint8), "wo_gscale": gscale,
               "wo_dequant_torch": lin.dequant_torch()}
        np.savez_compressed(os.path.join(HERE, "weights_nvfp4_rowscale.npz"), **to_np(out))
        print("wrote weights_nvfp4_rowscale")
    except Exception as e:  # pragma: no cover
        print("weights_nvfp4_rowscale skipped:", e)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
