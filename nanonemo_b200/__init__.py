"""nanonemo_b200: a Blackwell (sm_100a) native small-LM pretraining framework.

PyTorch is the framework layer (tensors, autograd, process groups, DCP); every hot
operator is a hand-written CUDA kernel in ``nanonemo_b200/csrc`` built ahead of time
into one shared library and reached through ``nanonemo_b200.ops``.
"""

__version__ = "0.1.0"
