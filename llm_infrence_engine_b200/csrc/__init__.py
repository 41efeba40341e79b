"""The CUDA library of the package: sources, build and the Python face of the kernels."""


def get_kernels():
    from .kernels import get_kernels as _get

    return _get()
