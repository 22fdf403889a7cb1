"""API types of the quantized-linear path: ActQuantizer / ActQuantWrapper with the attribute
contract of the reference (DiRotQ utils/quant_utils.py:88-106, :182-199, :286-323), plus the
module-wrapping helpers add_actquant / find_qlayers (:456-540).

These classes carry configuration only.  The arithmetic lives in the CUDA library; there is no
eager fake-quant here, so a wrapper whose forward has not been patched by
``dirotq_b200.backend.patch_forward`` refuses to run a quantised configuration.
"""
from __future__ import annotations

import torch
import torch.nn as nn


class ActQuantizer(nn.Module):
    """Configuration holder for the activation quantiser (same fields and ``configure`` signature
    as the reference class)."""

    def __init__(self):
        super().__init__()
        self.register_buffer("maxq", torch.tensor(0))
        self.bits = 16
        self.high_bits_length = 0
        self.groupsize = -1
        self.sym = False
        self.clip_ratio = 1.0
        self.quant_dtype = "int"

    def configure(self, bits, groupsize=-1, sym=False, clip_ratio=1.0, high_bits_length=0, quant_dtype="int"):
        self.quant_dtype = quant_dtype
        if quant_dtype == "nvfp4":
            sym = True
        self.maxq = torch.tensor(2 ** (bits - 1) - 1 if sym else 2 ** bits - 1)
        self.bits = bits
        self.groupsize = groupsize
        self.sym = sym
        self.clip_ratio = clip_ratio
        self.high_bits_length = high_bits_length

    def free(self):
        pass


class ActQuantWrapper(nn.Module):
    """Wraps one nn.Linear; same attributes as the reference wrapper."""

    def __init__(self, module: nn.Linear):
        super().__init__()
        self.module = module
        self.weight = module.weight
        self.bias = module.bias
        self.quantizer = ActQuantizer()
        self.rotation = None
        self.rotation_per_head = None
        self.num_heads = None
        self.head_dim = None
        self.use_hadamard = False
        self.hadamard_sign_flips = None
        self.hadamard_low_dim = None
        self.perm_idx = None

    def extra_repr(self):
        q = self.quantizer
        if q.bits >= 16:
            return "activations 16-bit"
        kind = "nvfp4" if q.quant_dtype == "nvfp4" else ("int%d %s" % (q.bits, "sym" if q.sym else "asym"))
        rot = "rotation" if self.rotation is not None else ("per-head rotation" if self.rotation_per_head is not None else
              ("hadamard" if self.use_hadamard else ("permutation" if self.perm_idx is not None else "no rotation")))
        return f"activations {kind}, group {q.groupsize}, {q.high_bits_length} channels kept 16-bit, {rot}"

    def forward(self, x):
        if self.quantizer.bits >= 16:
            return self.module(x)
        raise RuntimeError("ActQuantWrapper.forward is not patched: call dirotq_b200.backend.patch_forward() "
                           "(the quantised path has no eager fallback)")


def _match_skip(full_name, patterns):
    """'pat' substring, '^pat' prefix, 'pat$' suffix, '^pat$' exact."""
    for p in patterns:
        a0, a1 = p.startswith("^"), p.endswith("$")
        core = p[1 if a0 else 0: -1 if a1 else None]
        if (a0 and a1 and full_name == core) or (a0 and not a1 and full_name.startswith(core)) or \
           (a1 and not a0 and full_name.endswith(core)) or (not a0 and not a1 and core in full_name):
            return True
    return False


def add_actquant(module, name="", skip_names=None):
    """Recursively replace nn.Linear children by ActQuantWrapper (same traversal rules as the reference)."""
    skip_names = skip_names or []
    if isinstance(module, ActQuantWrapper):
        return
    for cname, child in list(module.named_children()):
        full = f"{name}.{cname}" if name else cname
        if isinstance(child, nn.Linear):
            if not _match_skip(full, skip_names):
                setattr(module, cname, ActQuantWrapper(child))
        elif isinstance(child, (nn.Sequential, nn.ModuleList)):
            for i, sub in enumerate(list(child.children())):
                sfull = f"{full}.{i}"
                if isinstance(sub, nn.Linear) and not _match_skip(sfull, skip_names):
                    child[i] = ActQuantWrapper(sub)
    for cname, child in module.named_children():
        add_actquant(child, f"{name}.{cname}" if name else cname, skip_names)


def find_qlayers(module, layers=None, name=""):
    layers = layers or [nn.Linear, ActQuantWrapper]
    if type(module) in layers:
        return {name: module}
    res = {}
    for cname, child in module.named_children():
        res.update(find_qlayers(child, layers, f"{name}.{cname}" if name else cname))
    return res
