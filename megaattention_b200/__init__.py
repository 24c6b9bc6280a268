"""B200 (sm_100a) implementation of one hot path: a single persistent prefill kernel that
runs causal varlen GQA FlashAttention, the row-parallel O_proj GEMM and the
tensor-parallel AllReduce on one shared 128-row tile.

``metadata`` is importable anywhere; ``runtime`` loads the CUDA shared library and fails
loudly when it is missing."""
