"""mythos_b200: a Blackwell (sm_100a) LLM training and inference framework with train-in-format
quantisation (OIL8 / OIL4 / I2_S), a byte-compatible ``.oil`` container, hand-written tcgen05
kernels and NVLink peer-memory collectives fused into compute kernels."""

__version__ = "0.1.0"
