"""elfa_b200 - a Blackwell (sm_100a) native LLM pre-training framework.

PyTorch is the framework layer (modules, autograd, process groups); one native library
(``elfa_b200/_native/libelfa_b200.so``, sources in ``elfa_b200/csrc``) holds the hand-written
kernels: tcgen05/TMEM/TMA GEMMs, attention, normalisation, cross-entropy, quantisation, optimizers
and the peer-memory communication kernels.
"""
__version__ = "0.1.0"
