"""CUDA kernels (sm_100a) behind a C ABI, and the Python operators that call them."""
