"""ctypes prototypes of the sm_100a kernel library's extern "C" launchers."""
import ctypes as C

V, I, L, F = C.c_void_p, C.c_int, C.c_long, C.c_float


def declare(lib):
    def sig(name, args, optional=False, restype=C.c_int):
        try:
            fn = getattr(lib, name)
        except AttributeError:
            if optional:
                return
            raise
        fn.restype = restype
        fn.argtypes = args

    sig("ronn_gemm", [V, V, V, V, V, I, I, I, I, I, I, I, I, I, I, V, V])
    sig("ronn_gemm_splitk", [V, V, V, I, I, I, I, I, I, I, I, V, V, V])
    sig("ronn_splitk_finalize", [V, I, V, V, V, V, V, V, L, I, F, I, I, I, V])
    sig("ronn_gemm_reduce", [V, V, I, I, I, I, I, V, V, L, V, I, I, I, I, V, L, V, V, L, C.c_double, I, I, V, V, V, F, I, V, V], optional=True)
    sig("ronn_argmax_exchange", [V, V, V, I, V, I, V, I, I, C.c_double, V, V], optional=True)
    sig("ronn_peer_reduce", [I, I, V, V, L, V, I, I, I, I, V, L, V, V, L, C.c_double, I, V, V, V, F, I, V, V], optional=True)
    sig("ronn_bitlinear_to_slot", [V, V, V, F, V, V, L, V, I, I, I, I, I, V, V], optional=True)
    sig("ronn_gemm_reduce_push", [V, V, I, I, I, I, I, V, V, L, V, I, I, I, I, V, L, V, V, L, C.c_double, I, I, V, V, V, F, I,
                                  V, L, L, V, V], optional=True)
    sig("ronn_ag_gemm", [V, I, V, I, V, I, V, I, I, I, I, I, V, V, I, C.c_double, I, I, V, V], optional=True)
    sig("ronn_signal_peers", [V, I, I, V], optional=True)
    sig("ronn_norm", [V, V, V, V, V, V, L, I, L, L, L, F, I, I, V])
    sig("ronn_softmax", [V, V, L, I, I, V])
    sig("ronn_softmax_strided", [V, V, L, I, L, I, V], optional=True)
    sig("ronn_set_rowwise_status", [V], optional=True)
    sig("ronn_unary", [V, V, L, I, I, V])
    sig("ronn_binary", [V, V, V, L, I, I, V])
    sig("ronn_swiglu_fused", [V, V, L, I, I, V])
    sig("ronn_fused_elementwise", [V, V, L, I, V, V, V, L, I, V], optional=True)
    sig("ronn_embedding", [V, V, V, V, V, L, I, I, I, L, I, V])
    sig("ronn_argmax", [V, V, V, L, I, L, I, I, V])
    sig("ronn_argmax_combine", [V, V, V, I, I, V])
    sig("ronn_sample", [V, L, I, L, V, V, I, V, V, V], optional=True)
    sig("ronn_cast", [V, V, L, I, I, V])
    sig("ronn_kv_append", [V, L, I, I, V, V, V, V, L, I, I, I, F, I, I, V])
    sig("ronn_paged_attention", [V, L, V, V, V, I, V, V, V, L, L, I, I, I, I, F, I, I, I, V, V, F, I, V, V, V])
    sig("ronn_gemm_rownorm", [V, V, V, V, V, V, V, V, I, I, I, I, I, I, F, I, I, V, V], optional=True)
    sig("ronn_fmha", [V, L, L, I, I, I, V, V, V, V, L, I, I, I, I, I, I, F, I, V, V])
    sig("ronn_fmha_paged", [V, L, L, I, V, V, L, V, I, V, V, V, V, V, L, I, I, I, I, I, I, F, I, V, V])
    sig("ronn_conv2d", [V, V, V, V, V, I, I, I, I, I, I, I, I, I, I, I, I, I, I, V, L, V, V], optional=True)
    sig("ronn_nchw_to_nhwc8", [V, V, I, I, I, I, I, V], optional=True)
    sig("ronn_nchw_to_s2d16", [V, V, I, I, I, I, I, V], optional=True)
    sig("ronn_maxpool_nhwc", [V, V, I, I, I, I, I, I, I, I, I, I, V], optional=True)
    sig("ronn_global_avgpool_nhwc", [V, V, I, I, I, I, V], optional=True)
    sig("ronn_act_quant_int8", [V, V, V, L, I, I, V], optional=True)
    sig("ronn_norm_quant_int8", [V, V, V, V, V, L, I, F, I, V], optional=True)
    sig("ronn_bitlinear", [V, V, V, F, V, V, V, I, I, I, I, I, V, V], optional=True)
    sig("ronn_bitlinear_workspace_bytes", [I, I, I], restype=L, optional=True)
    sig("ronn_swiglu_quant_int8", [V, V, V, L, I, I, V], optional=True)
    sig("ronn_ternary_pack", [V, V, L, I, V], optional=True)
