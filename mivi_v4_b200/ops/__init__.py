"""Python side of the CUDA kernels: build, load, argument checks, launches."""
