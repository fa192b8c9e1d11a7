"""B200-native routed-expert MoE layer: the reference's ``tensorfold.cuda.moe`` / ``experts`` / ``exl3.experts``
operator surface over a C-ABI library of hand-written sm_100a kernels."""

__version__ = "0.1.0"
