"""dirotq_b200: B200 (sm_100a) implementation of DiRotQ's quantized-linear inference path.

    from dirotq_b200.backend import patch_forward, preconvert_rotations_to_device

Modules: ops (torch front end of the C ABI), backend (drop-in forward), pack (weight packer host API),
rotation (stand-alone rotation), wrapper (ActQuantWrapper / ActQuantizer API types).
"""
__version__ = "0.1.0"
