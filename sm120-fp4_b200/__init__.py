"""B200-native (sm_100a) NVFP4 fused-MoE layer behind the operator surface of sm120fp4."""
__version__ = "0.1.0"
