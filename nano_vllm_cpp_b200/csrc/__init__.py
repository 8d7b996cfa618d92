"""Hand-written CUDA for sm_100a and its ctypes binding (``ops``)."""
