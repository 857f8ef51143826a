"""B200-native (sm_100a) gated-delta-net kernels behind the avelang_kernels calling convention."""
__version__ = "0.1.0"
