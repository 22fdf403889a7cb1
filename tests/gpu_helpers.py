"""Decoders from the device buffer layouts (include/dirotq_b200.h) to plain tensors, for parity tests."""
import torch

from oracle import dirotq_oracle as O
from dirotq_b200 import ops


def decode_act(buf: ops.ActBuffers):
    """-> dict(codes [M, G, gs] int16, scale [M, G], zero [M, G] or None, tail [M, tail_total])."""
    lay, fmt, M = buf.layout, buf.fmt, buf.M
    ldm = buf.ldm
    raw = buf.codes.cpu()[: M * lay.code_row_bytes].reshape(M, lay.code_row_bytes)
    out = {}
    if fmt.mode in (ops.NVFP4_REF, ops.NVFP4_HW):
        nib = O.unpack_seq_nibbles(raw)[:, : lay.n_groups * 16]
        out["codes"] = nib.reshape(M, lay.n_groups, 16)
        if fmt.mode == ops.NVFP4_REF:
            s = buf.scales.cpu()[: lay.n_scales * ldm * 2].view(torch.bfloat16).reshape(lay.n_scales, ldm)
            out["scale"] = s[:, :M].T.contiguous()
        else:
            sfb = O.sf_untile(buf.scales.cpu(), M, lay.n_chunks * 4)[:, : lay.n_groups]
            out["scale_bytes"] = sfb
            out["scale"] = sfb.view(torch.float8_e4m3fn).float()
    else:
        if fmt.mode == ops.INT8_ASYM:
            c = raw.to(torch.int16)
        else:
            c = O.unpack_planar32(raw, signed=(fmt.mode == ops.INT4_SYM))
        cpg = lay.chunks_per_group
        c = c.reshape(M, lay.n_groups, cpg * 64)
        out["codes_padded"] = c
        out["codes"] = c[:, :, : lay.group]
        s = buf.scales.cpu()[: lay.n_scales * ldm * 2].view(torch.bfloat16).reshape(lay.n_scales, ldm)
        out["scale_chunks"] = s[:, :M].T.contiguous()
        out["scale"] = out["scale_chunks"][:, ::cpg].contiguous()
        if buf.zeros is not None:
            z = buf.zeros.cpu()[: lay.n_scales * ldm * 2].view(torch.bfloat16).reshape(lay.n_scales, ldm)
            out["zero"] = z[:, :M].T[:, ::cpg].contiguous()
    if buf.tail is not None:
        t = buf.tail.cpu()[: M * lay.tail_pitch * 2].view(torch.bfloat16).reshape(M, lay.tail_pitch)
        out["tail"] = t[:, : lay.tail_total].contiguous()
    return out


def oracle_cfg(fmt: ops.ActFormat, lay: ops.ActLayout) -> O.QuantCfg:
    """QuantCfg the reference quantiser sees for this format (after the per-head override)."""
    if fmt.mode in (ops.NVFP4_REF, ops.NVFP4_HW):
        return O.QuantCfg(4, 16, True, fmt.clip_ratio, lay.tail_total, "nvfp4")
    bits = 8 if fmt.mode == ops.INT8_ASYM else 4
    group = -1 if (fmt.num_heads == 0 and fmt.group_size <= 0) else lay.group      # per-token scales
    return O.QuantCfg(bits, group, fmt.mode == ops.INT4_SYM, fmt.clip_ratio, lay.tail_total, "int")


def to_reference_layout(x_rot2d: torch.Tensor, fmt: ops.ActFormat) -> torch.Tensor:
    """[M, D] in the wrapper's layout -> [1, M, D] in the layout the reference quantiser is fed
    (per-head: [H*d_q | H*hlen], dirotq_fused_unrotation_fast.py:83-88)."""
    x = x_rot2d.cpu()
    if fmt.num_heads > 0:
        x = O.per_head_rearrange(x.reshape(x.shape[0], fmt.num_heads, fmt.head_dim), fmt.tail_len)
    return x.unsqueeze(0)


def assert_act_matches_oracle(buf: ops.ActBuffers, x_rot2d: torch.Tensor):
    """Bit-exact comparison of codes / scales / zeros / tail with the oracle on the same rotated tensor."""
    fmt, lay = buf.fmt, buf.layout
    dec = decode_act(buf)
    xin = to_reference_layout(x_rot2d, fmt)
    cfg = oracle_cfg(fmt, lay)
    if fmt.mode == ops.NVFP4_HW:
        r = O.act_quant_nvfp4_hw(xin, cfg, fmt.tensor_scale)
    else:
        r = O.act_quant(xin, cfg)
    M = buf.M
    ref_codes = r.codes.reshape(M, lay.n_groups, -1)
    got = dec["codes"]
    # padded slots of a partial last group carry no information in the reference (trimmed)
    valid = torch.ones_like(ref_codes, dtype=torch.bool)
    rem = lay.q_len - (lay.n_groups - 1) * lay.group
    if rem < lay.group:
        valid[:, -1, rem:] = False
    assert got.shape == ref_codes.shape, (got.shape, ref_codes.shape)
    bad = ((got.to(torch.int16) != ref_codes.to(torch.int16)) & valid)
    assert not bool(bad.any()), f"{int(bad.sum())} code mismatches of {bad.numel()}"
    ref_scale = r.scale.reshape(M, lay.n_groups)
    if fmt.mode == ops.NVFP4_HW:
        assert torch.equal(dec["scale"], ref_scale.float()), "scale-factor mismatch"
    else:
        assert torch.equal(dec["scale"].view(torch.int16), ref_scale.contiguous().view(torch.int16)), "scale mismatch"
    if r.zero is not None:
        assert torch.equal(dec["zero"].view(torch.int16), r.zero.reshape(M, lay.n_groups).contiguous().view(torch.int16))
    if lay.tail_total > 0:
        assert torch.equal(dec["tail"].view(torch.int16), r.tail.reshape(M, -1).contiguous().view(torch.int16))
    return dec, r


def dense_reference_weight(w, ld) -> torch.Tensor:
    """fp32 [N, D] fused weight, in the layout nn.Linear holds in the reference ([Q(low) | tail];
    per head: [low_h | tail_h] for every head), rebuilt from the explicit codes a synthetic layer carries."""
    ex = w._b200_explicit
    N = ld.out_f
    if "nibbles" in ex:
        vals = torch.tensor(O.E2M1_VALUES)
        nib = ex["nibbles"].cpu().long()
        mag = vals[nib & 7] * torch.where((nib & 8) != 0, -1.0, 1.0)
        sc = ex["scales_e4m3"].cpu().view(torch.float8_e4m3fn).float() * ex["tensor_scale"]
        low = (mag.reshape(N, -1, 16) * sc.unsqueeze(-1)).reshape(N, -1)
    else:
        codes = ex["codes"].cpu().float()
        sc = ex["scales"].cpu().float()
        G = sc.shape[1]
        gs = (ld.head_dim - ld.tail) if ld.kind == "perhead" else 64
        pad = G * gs - codes.shape[1]
        if pad:
            codes = torch.nn.functional.pad(codes, (0, pad))
        low = (codes.reshape(N, G, gs) * sc.unsqueeze(-1)).reshape(N, -1)[:, : ex["codes"].shape[1]]
    tail = ex.get("w_tail")
    if tail is None:
        return low
    tail = tail.cpu().float().to(torch.bfloat16).float()
    if ld.kind == "perhead":
        H, d, hl = ld.heads, ld.head_dim, ld.tail
        return torch.cat([low.reshape(N, H, d - hl), tail.reshape(N, H, hl)], dim=2).reshape(N, H * d)
    return torch.cat([low, tail], dim=1)
