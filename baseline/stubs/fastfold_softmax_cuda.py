"""Import placeholder for the reference's CUDA softmax extension.

The reference imports this module unconditionally but only calls it when
Triton is not importable; with Triton present its own Triton kernels run.  The
extension itself does not build against this PyTorch (it is compiled with
``-std=c++14`` and includes a header PyTorch no longer ships).
"""


def __getattr__(name):
    raise RuntimeError("fastfold_softmax_cuda is not built on this machine (Triton path expected)")
