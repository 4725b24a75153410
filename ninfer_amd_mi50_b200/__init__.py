"""A small, whole inference engine for one B200: Qwen2-MoE from a model folder to tokens.

Shaped after NInfer-HIP (srmmushi/Ninfer-AMD-Mi50): configuration, weights, parts, cache,
step function, scheduler, sampling, command line and Python entry point, with
hand-written CUDA for sm_100a underneath.
"""

__version__ = "0.1.0"
