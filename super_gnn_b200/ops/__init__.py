from .spmm_kernel import SPMM_forward, SPMM_backward  # noqa: F401
