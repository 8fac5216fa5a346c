"""The compiled pybind11 form of the operator module (`_cuda_ops`, built from csrc/bindings_pybind.cc by
`python ac4k_kernel_b200/build.py --pybind`): the same names and positional signatures as the reference's
`ac4k_kernel._cuda_ops` (lib/cuda_bindings.cc:37-97).  `ac4k_kernel_b200._cuda_ops` is the ctypes form of the
same interface; both call the same C ABI."""


def load():
    """Import and return the compiled module; raises ImportError with the build command if it is not built."""
    try:
        from . import _cuda_ops
    except ImportError as e:
        raise ImportError("the pybind module is not built: run `python ac4k_kernel_b200/build.py --pybind`") from e
    return _cuda_ops
