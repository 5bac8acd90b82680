"""autoresearch_b200: a Blackwell-native GPT pre-training engine.

Layers: cli -> config -> trainer -> models / optim / parallel / data / ckpt / eval -> ops
(sm_100a CUDA kernels) and native (C++ host library).
"""
__version__ = "0.1.0"
