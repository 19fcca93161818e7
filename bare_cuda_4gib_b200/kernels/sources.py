"""The CUDA libraries of the engine: (source file, -D flags) pairs.  A model compiles what it
needs at first use; `all_libraries()` is everything, for the build check."""

ATTENTION_HEAD_DIMS = (16, 32, 48, 64, 80, 96, 112, 128)
# (entries of one map, value entries) of differential attention on the tensor cores, as the presets have them
DIFF_ATTENTION_SIZES = ((16, 16), (64, 128), (128, 256))


def all_libraries():
    jobs = [("plain_kernels.cu", ()), ("gemm_tcgen05.cu", ()), ("gemv_fused.cu", ()), ("stream_kernels.cu", ()),
            ("linear_attention.cu", ()), ("biased_attention.cu", ()), ("sandwich_norm.cu", ()), ("head_prepare.cu", ()),
            ("latent_attention.cu", ()), ("mlstm.cu", ()), ("diff_attention.cu", ()), ("moe.cu", ()),
            ("gated_sandwich.cu", ()), ("mamba2.cu", ()),
            ("mamba2_chunked.cu", ("-DSSD_N=128", "-DSSD_P=64", "-DSSD_PC=16")),
            ("mamba2_chunked.cu", ("-DSSD_N=128", "-DSSD_P=64", "-DSSD_PC=32"))]
    jobs += [("gemm_tcgen05.cu", ("-DGLU_GELU_TANH",)), ("gemv_fused.cu", ("-DGLU_GELU_TANH",)),
             ("gemm_tcgen05.cu", ("-DGROUPED_UP_RELU2",))]
    jobs += [("attention_mma.cu", (f"-DHEAD_DIM={d}",)) for d in ATTENTION_HEAD_DIMS]
    jobs += [("attention_mma.cu", (f"-DHEAD_DIM={d}", "-DDISTANCE_BIAS")) for d in ATTENTION_HEAD_DIMS]
    # value heads of their own size and capped scores, as the Gurolix presets have them
    jobs += [("attention_mma.cu", ("-DHEAD_DIM=128", "-DV_DIM=64")), ("attention_mma.cu", ("-DHEAD_DIM=128", "-DV_DIM=64", "-DSCORE_CAP")),
             ("attention_mma.cu", ("-DHEAD_DIM=128", "-DSCORE_CAP")), ("attention_mma.cu", ("-DHEAD_DIM=16", "-DV_DIM=32", "-DSCORE_CAP"))]
    jobs += [("attention_tcgen05.cu", (f"-DHEAD_DIM={d}",)) for d in (64, 128)]
    jobs += [("attention_decode.cu", (f"-DHEAD_DIM={d}",)) for d in (64, 128)]
    jobs += [("diff_attention.cu", (f"-DDA_DQ={d}", f"-DDA_DV={v}")) for d, v in DIFF_ATTENTION_SIZES]
    return jobs
