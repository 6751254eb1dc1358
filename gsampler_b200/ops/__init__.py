from .spmm import gspmm
from .sddmm import gsddmm
from .fused import e_square_sum, e_div_u_sum

__all__ = ["gspmm", "gsddmm", "e_square_sum", "e_div_u_sum"]
