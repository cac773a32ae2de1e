"""Python bindings of the package's CUDA kernels (`ops`)."""
