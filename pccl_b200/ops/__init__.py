"""Hand-written sm_100a operators (tcgen05 GEMMs, fused epilogues, collectives, quantisers)."""
from .gemm import gemm, gemm_nn, gemm_nt, gemm_tn, launch_count, status_words, check_status

__all__ = ["gemm", "gemm_nn", "gemm_nt", "gemm_tn", "launch_count", "status_words", "check_status"]
