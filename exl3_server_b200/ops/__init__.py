"""The CUDA kernel library and its Python faces."""
