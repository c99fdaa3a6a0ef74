"""Hand-written CUDA kernels for sm_100a and their Python table (``ops``)."""
