"""CUDA kernels for sm_100a: build system (``build``) and Python entry points (``ops``)."""
