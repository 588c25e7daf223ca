"""The CUDA kernels: ``build`` compiles them, ``ops`` calls them."""
