"""Case table shared by the fixture generator (make_golden.py) and the tests.

Einsummable cases: (name, einsum string, extents, join, castable, input range).
`join` is either the reference's text form or ("builder", dtype) resolved by the
generator through the reference's own scalarop_t::make_* functions and stored
in golden.json.  Shapes follow the kernel cases of the reference's
exps/gpuexec_kernelmanager.cc (reduced where the interpreter would take
minutes) and the einsummables one LLaMA layer emits (llama/modules.cc).
"""

B = lambda name, dt: ("builder", name, dt)

EINSUMMABLE_CASES = [
    # --- contractions (exps/gpuexec_kernelmanager.cc:41,432-948,3129-3132) ---
    ("mm_f64_golden_shape", "ij,jk->ik", dict(i=3, j=4, k=5), B("mul", "f64"), "add", (-1, 1)),
    ("mm_ss_f32", "ij,jk->ik", dict(i=24, j=40, k=16), B("mul", "f32"), "add", (-1, 1)),
    ("mm_st_f16", "ij,kj->ik", dict(i=16, j=32, k=24), B("mul", "f16"), "add", (-1, 1)),
    ("mm_ts_f32", "ji,jk->ik", dict(i=8, j=12, k=20), B("mul", "f32"), "add", (-1, 1)),
    ("mm_tt_f16", "ji,kj->ik", dict(i=8, j=16, k=8), B("mul", "f16"), "add", (-1, 1)),
    ("contraction_5mode_f32", "adbe,dec->abc", dict(a=3, b=4, c=5, d=2, e=6), B("mul", "f32"), "add", (-1, 1)),
    ("attn_scores_f16", "acbe,adbe->abcd", dict(a=2, b=3, c=8, d=8, e=16), B("mul", "f16"), "add", (-1, 1)),
    ("attn_pv_f16", "abce,aebd->abcd", dict(a=2, b=3, c=8, d=16, e=8), B("mul", "f16"), "add", (-1, 1)),
    ("attn_wo_f16", "aebf,cdef->abcd", dict(a=2, b=4, c=3, d=8, e=3, f=8), B("mul", "f16"), "add", (-1, 1)),
    ("contraction_c64", "ij,jk->ik", dict(i=4, j=6, k=5), B("mul", "c64"), "add", (-1, 1)),
    ("dot_1d_f32", "a,a->a", dict(a=50), B("mul", "f32"), None, (-1, 1)),
    # --- reductions (:1399-1643,3284) ---
    ("sum_ab_a_f32", "ab->a", dict(a=7, b=100), B("identity", "f32"), "add", (-1, 1)),
    ("sum_ab_a_f16", "ab->a", dict(a=5, b=64), B("identity", "f16"), "add", (-1, 1)),
    ("max_ab_a_f32", "ab->a", dict(a=9, b=33), B("identity", "f32"), "max", (-5, 5)),
    ("max_ab_a_f16", "ab->a", dict(a=6, b=48), B("identity", "f16"), "max", (-5, 5)),
    ("min_ab_a_f64", "ab->a", dict(a=4, b=21), B("identity", "f64"), "min", (-5, 5)),
    ("prod_ab_a_f32", "ab->a", dict(a=6, b=12), B("identity", "f32"), "mul", (0.5, 1.5)),
    ("negsum_ab_a_f32", "ab->a", dict(a=6, b=40), B("neg", "f32"), "add", (-1, 1)),
    ("colsum_ba_a_f32", "ba->a", dict(a=37, b=19), B("identity", "f32"), "add", (-1, 1)),
    ("colmax_ba_a_f16", "ba->a", dict(a=40, b=10), B("identity", "f16"), "max", (-5, 5)),
    ("sum_abc_b_f32", "abc->b", dict(a=5, b=6, c=8), B("identity", "f32"), "add", (-1, 1)),
    ("sum_c64", "ab->a", dict(a=4, b=10), B("identity", "c64"), "add", (-1, 1)),
    ("softmax_v3_sum_f32", "ab,a->a", dict(a=6, b=64), B("softmax_v3_sum:0.0883883", "f32"), "add", (-2, 2)),
    ("exp_sub_sum_f32", "ab,a->a", dict(a=8, b=40), B("exp_sub", "f32"), "add", (-2, 2)),
    ("large_workspace_1_f32", "ab,ab,a->a", dict(a=5, b=32),
     "*[hole|f32@0,*[hole|f32@1,*[constant{f32|-1},power{-2}[hole|f32@2]]]]", "add", (0.5, 2)),
    # --- elementwise (:1656-2021,2040-2582,2959-3354) ---
    ("silu_f16", "a->a", dict(a=200), B("silu", "f16"), None, (-4, 4)),
    ("silu_f32", "a->a", dict(a=200), B("silu", "f32"), None, (-4, 4)),
    ("silu_mul_f16", "a,a->a", dict(a=256), B("silu_mul", "f16"), None, (-4, 4)),
    ("silu_mul_f32", "a,a->a", dict(a=96), B("silu_mul", "f32"), None, (-4, 4)),
    ("exp_sub_rowmax_f16", "ab,a->ab", dict(a=6, b=40), B("exp_sub", "f16"), None, (-3, 3)),
    ("exp_sub_rowmax_f32", "ab,a->ab", dict(a=6, b=36), B("exp_sub", "f32"), None, (-3, 3)),
    ("square_f32", "a->a", dict(a=100), B("square", "f32"), None, (-3, 3)),
    ("invsqrt_f32", "a->a", dict(a=100), B("inverse_sqrt", "f32"), None, (0.1, 9)),
    ("sqrt_f64", "a->a", dict(a=33), B("sqrt", "f64"), None, (0.1, 9)),
    ("power3_f32", "a->a", dict(a=64), B("power:3", "f32"), None, (-2, 2)),
    ("exp_f32", "a->a", dict(a=128), B("exp", "f32"), None, (-5, 5)),
    ("log_f32", "a->a", dict(a=64), B("log", "f32"), None, (0.1, 20)),
    ("relu_f32", "a->a", dict(a=77), B("relu", "f32"), None, (-3, 3)),
    ("relu_f16", "a->a", dict(a=80), B("relu", "f16"), None, (-3, 3)),
    ("sigmoid_f32", "a->a", dict(a=64), B("sigmoid", "f32"), None, (-6, 6)),
    ("scale_f16", "a->a", dict(a=64), B("scale:0.25", "f16"), None, (-3, 3)),
    ("rms_eps_scale_f32", "a->a", dict(a=48), "+[constant{f32|1e-06},*[constant{f32|0.000244141},hole|f32@0]]",
     None, (0, 4000)),
    ("to_f32", "a->a", dict(a=120), B("convert:f32", "f16"), None, (-9, 9)),
    ("to_f16", "a->a", dict(a=120), B("convert:f16", "f32"), None, (-9, 9)),
    ("to_f64", "a->a", dict(a=30), B("convert:f64", "f32"), None, (-9, 9)),
    ("f64_to_f32", "a->a", dict(a=30), B("convert:f32", "f64"), None, (-9, 9)),
    ("add_aa_f16", "a,a->a", dict(a=136), B("add", "f16"), None, (-3, 3)),
    ("mul_aa_f16", "a,a->a", dict(a=72), B("mul", "f16"), None, (-3, 3)),
    ("add_ab_b_f32", "ab,b->ab", dict(a=6, b=20), B("add", "f32"), None, (-3, 3)),
    ("mul_ab_b_f16", "ab,b->ab", dict(a=5, b=24), B("mul", "f16"), None, (-3, 3)),
    ("mul_ab_a_f32", "ab,a->ab", dict(a=7, b=12), B("mul", "f32"), None, (-3, 3)),
    ("div_ab_a_f32", "ab,a->ab", dict(a=7, b=16), B("div", "f32"), None, (0.5, 3)),
    ("sub_ab_a_f32", "ab,a->ab", dict(a=7, b=9), B("sub", "f32"), None, (-3, 3)),
    ("max_aa_f32", "a,a->a", dict(a=50), B("max", "f32"), None, (-3, 3)),
    ("min_aa_f16", "a,a->a", dict(a=50), B("min", "f16"), None, (-3, 3)),
    ("is_equal_ab_a_f32", "ab,a->ab", dict(a=4, b=8), B("is_equal", "f32"), None, "ints"),
    ("large_workspace_2_f32", "ab,a,a->ab", dict(a=6, b=10),
     "*[*[hole|f32@0,power{-1}[hole|f32@1]],hole|f32@2]", None, (0.5, 3)),
    ("softmax_v3_norm_f32", "ab,a,a->ab", dict(a=5, b=24), B("softmax_v3_norm:0.0883883", "f32"), None, (0.5, 3)),
    ("rope_c64", "abcd,bd->abcd", dict(a=2, b=5, c=3, d=4), B("mul", "c64"), None, (-1, 1)),
    ("conj_c64", "a->a", dict(a=20), B("conjugate", "c64"), None, (-1, 1)),
    ("real_c64", "a->a", dict(a=20), B("project_real", "c64"), None, (-1, 1)),
    ("complex_f32", "a,a->a", dict(a=20), B("complex", "c64"), None, (-1, 1)),
    ("add_f64", "a,a->a", dict(a=33), B("add", "f64"), None, (-3, 3)),
    ("axpby_f32", "a,a->a", dict(a=40), "+[*[constant{f32|0.5},hole|f32@0],*[constant{f32|-500},hole|f32@1]]",
     None, (-1, 1)),
    # --- permutations / broadcasts (identity join) ---
    ("perm_bhsd_bshd_f16", "acbd->abcd", dict(a=2, b=6, c=3, d=8), B("identity", "f16"), None, (-3, 3)),
    ("transpose_ba_ab_f32", "ba->ab", dict(a=37, b=45), B("identity", "f32"), None, (-3, 3)),
    ("transpose_cba_f16", "cba->abc", dict(a=5, b=6, c=33), B("identity", "f16"), None, (-3, 3)),
    ("transpose_silu_f32", "ba->ab", dict(a=20, b=35), B("silu", "f32"), None, (-3, 3)),
    ("transpose_add_f32", "ba,ab->ab", dict(a=20, b=33), B("add", "f32"), None, (-3, 3)),
    ("broadcast_b_ab_f32", "b->ab", dict(a=6, b=10), B("identity", "f32"), None, (-3, 3)),
    ("broadcast_a_ab_f16", "a->ab", dict(a=6, b=16), B("identity", "f16"), None, (-3, 3)),
    ("perm_c64", "ba->ab", dict(a=6, b=7), B("identity", "c64"), None, (-3, 3)),
]

# merge_adjacent_dims / str cases: (join_shape, inns, out_rank)
MERGE_CASES = [
    ([4, 512, 32, 128, 32, 128], [[0, 4, 1, 5], [2, 3, 4, 5]], 4),   # WO: aebf,cdef->abcd
    ([4, 512, 32, 128, 4096], [[0, 1, 4], [2, 3, 4]], 4),            # QKV: abef,cdef->abcd style
    ([4, 32, 512, 512, 128], [[0, 2, 1, 4], [0, 3, 1, 4]], 4),       # scores
    ([4, 32, 512, 128, 512], [[0, 1, 2, 4], [0, 4, 1, 3]], 4),       # P.V
    ([4, 512, 32, 64], [[0, 1, 2, 3], [1, 3]], 4),                   # rope
    ([4, 512, 4096], [[0, 1, 2], [0, 1, 2]], 3),                     # straight binary
    ([4, 512, 4096], [[0, 1, 2], [2]], 3),                           # ab,b->ab
    ([4, 512, 4096], [[0, 1, 2], [0, 1]], 3),                        # ab,a->ab
    ([4, 512, 4096], [[0, 1, 2]], 2),                                # ab->a
    ([32, 512, 32, 128], [[0, 2, 1, 3]], 4),                         # bhsd<->bshd
    ([3, 5, 4], [[0, 2], [2, 1]], 2),
    ([8, 6, 4, 2], [[3, 2, 1, 0]], 4),
    ([8, 6, 4, 2], [[0, 1, 2, 3], [2, 3]], 2),
    ([2, 3, 4, 5, 6], [[0, 1, 3, 4], [3, 4, 2]], 3),
]

TOUCH_DTYPES = ["f16", "f32", "f64", "c64"]
TOUCH_CASTABLES = [None, "add", "mul", "min", "max"]

FILL_CASES = [
    # (dtype, lower, upper, nrow, ncol, start)
    ("f16", 0.0, float("-inf"), 16, 16, 0),
    ("f32", 1.0, 0.0, 7, 12, 3),
    ("f32", 1.0, 0.0, 12, 7, -4),
    ("f64", 2.5, -1.0, 5, 5, 9),
    ("f16", 1.0, 0.0, 6, 9, -20),
    ("c64", 1 + 2j, 0j, 4, 6, 1),
]
