"""ctypes signatures of the CUDA library's C entry points."""
from ctypes import c_float, c_int, c_int64, c_size_t, c_void_p


def declare(lib):
    P, I, L, F = c_void_p, c_int, c_int64, c_float
    lib.ft_adam_cuda.argtypes = [P, P, I, P, P, P, I, L, L, F, F, F, F, F, I, I, F, P, P]
    lib.ft_check_finite.argtypes = [P, I, L, P, P]
    lib.ft_accumulate_zero.argtypes = [P, I, P, I, L, P]
    lib.ft_cast_copy.argtypes = [P, I, P, I, L, P]
    lib.ft_pinned_alloc.restype = c_void_p
    lib.ft_pinned_alloc.argtypes = [c_size_t]
    lib.ft_pinned_free.argtypes = [P]
    lib.ft_rmsnorm_fwd.argtypes = [P, P, P, P, L, I, F, I, P]
    lib.ft_rmsnorm_bwd_parts.restype = I
    lib.ft_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, L, I, I, P]
    lib.ft_norm_max_hidden.argtypes = [I]
    lib.ft_norm_max_hidden.restype = I
    lib.ft_norm_bwd_parts.argtypes = [L, I]
    lib.ft_norm_bwd_parts.restype = I
    lib.ft_norm_fwd.argtypes = [P, P, P, P, P, P, L, I, F, I, I, P]
    lib.ft_norm_bwd.argtypes = [P, P, P, P, P, P, P, P, P, P, L, I, I, I, P]
    lib.ft_add_norm_fwd.argtypes = [P, P, P, P, P, P, P, P, L, I, F, I, I, P]
    lib.ft_add_norm_bwd.argtypes = [P, P, P, P, P, P, P, P, P, P, P, L, I, I, I, P]
    lib.ft_bias_act_fwd.argtypes = [P, P, P, L, I, I, I, P]
    lib.ft_bias_act_bwd_parts.argtypes = [L, I]
    lib.ft_bias_act_bwd_parts.restype = I
    lib.ft_bias_act_bwd.argtypes = [P, P, P, P, P, P, L, I, I, I, I, P]
    lib.ft_rope.argtypes = [P, L, P, L, P, P, L, I, I, I, F, I, P]
    lib.ft_swiglu_fwd.argtypes = [P, P, L, I, I, P]
    lib.ft_swiglu_bwd.argtypes = [P, P, P, L, I, I, P]
    lib.ft_xent_fwd.argtypes = [P, L, P, L, I, L, P, P, I, P]
    lib.ft_xent_bwd.argtypes = [P, L, P, L, I, L, P, P, F, I, P]
    lib.ft_count_valid.argtypes = [P, L, L, I, P, P]
    lib.ft_gemm.argtypes = [P, I, L, P, I, L, P, L, I, I, I, I, I, I, P]
    lib.ft_gemm_add.argtypes = [P, I, L, P, I, L, P, L, I, I, P, L, I, I, I, I, P]
    lib.ft_gemm_add.restype = I
    lib.ft_gemm_swiglu.argtypes = [P, L, P, L, P, L, P, L, I, I, I, I, P]
    lib.ft_gemm_error.restype = I
    lib.ft_launch_count.restype = c_int64
    for name in ("ft_attn_fwd", "ft_attn_bwd"):
        if hasattr(lib, name):
            getattr(lib, name).restype = I
