"""Bindings of the hand-written CUDA kernels (``functional``) and their loader (``library``)."""
