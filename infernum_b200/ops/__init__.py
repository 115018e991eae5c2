"""ctypes wrappers over the package's CUDA kernel modules."""
