"""B200-native Kimi Delta Attention: hand-written sm_100a kernels behind a C ABI
(include/kda_b200.h) and a host-side mirror of the reference mixer interface."""

from .kda import (KDAState, KimiDeltaAttention, RMSNormGated, ShortConvolution, chunk_kda, chunk_kda_norm, k3_decay_gate, kda,
                  kda_backend_provenance, prepare_kda_backend, recurrent_kda_step, short_convolutions)

__all__ = ["KDAState", "KimiDeltaAttention", "RMSNormGated", "ShortConvolution", "chunk_kda", "chunk_kda_norm", "k3_decay_gate", "kda",
           "kda_backend_provenance", "prepare_kda_backend", "recurrent_kda_step", "short_convolutions"]
