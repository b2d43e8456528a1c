"""thundersvm_b200: B200 (sm_100a) implementation of ThunderSVM's batched-SMO / KernelMatrix /
prediction hot path behind a C ABI (include/thundersvm_b200.h)."""
__all__ = ["capi", "synth", "build"]
