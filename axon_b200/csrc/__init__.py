"""Native sources (CUDA kernels, host library) and their in-tree build."""
