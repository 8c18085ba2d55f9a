"""Which kernels the library may choose among, fixed when an engine is built.

Every field at its default leaves the choice to the measured dispatch rules of the kernel library; the other
values pin one path (tests hold each path against the plain references, benchmarks compare them). The set is
frozen: an engine carries its own in its ``EngineConfig``, two engines in one process do not see each other's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_ROUTES = (None, "smallm", "smallm_fused", "tc", "tc_pair")


@dataclass(frozen=True)
class KernelOptions:
    force_general_attention: bool = False   # the general (CUDA-core) attention kernel for bfloat16 too
    force_mma_prefill: bool = False         # prompt portions on the mma.sync attention kernel instead of tcgen05
    decode_tma: bool = True                 # decode attention with TMA page loads where the shape allows (else mma.sync + cp.async)
    separate_combine: bool = True           # cp.async decode kernel: merge its splits in a second kernel (False: the CTA that finishes last merges)
    fixed_decode_splits: int = 0            # a fixed split count of the keys for the decode kernels (0 = chosen)
    force_simt_gemm: bool = False           # the CUDA-core product for bfloat16 too
    gemm_route: Optional[str] = None        # "smallm" | "smallm_fused" | "tc" | "tc_pair" instead of the measured choice
    tc_token_tile: int = 0                  # token tile of the tcgen05 product (0 = chosen; 16, 32, 64, 128, 256)
    tc_splits: int = 0                      # work items along K per tile of the tcgen05 products (0 = chosen, 1 = none)
    pair_n_tile: int = 0                    # feature tile of the two-SM product (0 = chosen; 128, 256)
    smallm_ksplit: int = 0                  # K split among the warps of a CTA in the small-M product (0 = chosen; 1, 8)
    smallm_cross: int = 0                   # CTAs that split K further in the small-M product (0 = chosen)
    fuse_qkv: bool = True                   # up to 16 tokens: bias, rotation and the page write are the q/k/v product's epilogue

    def __post_init__(self):
        if self.gemm_route not in _ROUTES:
            raise ValueError(f"gemm_route must be one of {_ROUTES}, got {self.gemm_route!r}")
        for name in ("fixed_decode_splits", "tc_token_tile", "tc_splits", "pair_n_tile", "smallm_ksplit", "smallm_cross"):
            if getattr(self, name) < 0:
                raise ValueError(f"{name} must be >= 0")
