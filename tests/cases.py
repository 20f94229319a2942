"""Shared parity-case table: one description of (operator, arguments, seeded inputs) that the
golden-fixture generator, the oracle tests and the GPU parity tests all iterate over.

A case is a dict: ``name``, ``op`` (operator type string), ``args`` (operator arguments, the
reference's names), ``inputs`` (list of float32 arrays: the operator's bottoms in order).
Input tensors are seeded ``numpy.random.Generator(PCG64(seed))`` draws cast to float32.
"""
from __future__ import annotations

import numpy as np

from oracle import oracle as orc

SPECIALS = np.array(
    [0.0, -0.0, 1.0, -1.0, np.nan, np.inf, -np.inf, 3.4028235e38, -3.4028235e38, 1.17549435e-38,
     1e-45, -1e-45, 0.5, -0.5, 2.0, 3.0, -3.0, 6.0, 6.5, -7.25, 88.0, -88.0, 104.0, -104.0,
     0.33333334, 1e-3, 16.0, 1e10, -1e10, 9.5, 2.5, -2.5], dtype=np.float32)


GOLDEN_FULL_LIMIT = 65536   # outputs larger than this are pinned by SHA-256 digest in the fixture


def golden_lookup(golden, name):
    """(array or None, digest or None, shape) for a case of tests/golden/small_cases.npz."""
    shape = [int(d) for d in golden[name + "/shape"]]
    if name in golden.files:
        return golden[name], None, shape
    return None, bytes(golden[name + "/sha256"]), shape


def rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def uniform(seed, shape, lo=-1.0, hi=1.0):
    return rng(seed).uniform(lo, hi, size=shape).astype(np.float32)


def normal(seed, shape, mean=0.0, std=1.0):
    return rng(seed).normal(mean, std, size=shape).astype(np.float32)


def _case(name, op, args, inputs, n_tops=1):
    c = {"name": name, "op": op, "args": args, "inputs": [np.ascontiguousarray(x, np.float32) for x in inputs]}
    if n_tops != 1:
        c["n_tops"] = n_tops   # several outputs: results are compared flattened, one after another
    return c


def special_pairs():
    """Every ordered pair of special values, as two flat arrays."""
    a, b = np.meshgrid(SPECIALS, SPECIALS, indexing="ij")
    return a.ravel().copy(), b.ravel().copy()


def small_cases():
    """Cases the C oracle finishes in well under a second each; covers every operation code of
    the six operators, ragged sizes, every broadcast position, rank padding, edge values."""
    cs = []
    # ---- Binary: same shape, scalar, broadcast --------------------------------------------
    for opname, code in orc.BINARY.items():
        lo = 0.1 if opname == "Pow" else -2.0
        a = uniform(100 + code, (3, 5, 7, 11), lo, 2.0)
        b = uniform(200 + code, (3, 5, 7, 11), lo, 2.0)
        cs.append(_case("binary_same_%s" % opname, "Binary", {"operation": code}, [a, b]))
        cs.append(_case("binary_scalar_%s" % opname, "Binary",
                        {"operation": code, "scalar": float(np.float32(0.7))}, [a]))
        cs.append(_case("binary_bcast_chan_%s" % opname, "Binary", {"operation": code},
                        [a, uniform(300 + code, (1, 5, 1, 1), lo, 2.0)]))
    sa, sb = special_pairs()
    for opname in ("Add", "Sub", "Mul", "Div", "Max", "Min"):
        cs.append(_case("binary_special_%s" % opname, "Binary", {"operation": orc.BINARY[opname]}, [sa, sb]))
    for sc in (0.0, -0.0, float("nan"), float("inf")):
        for opname in ("Max", "Min", "Mul"):
            cs.append(_case("binary_scalar_special_%s_%r" % (opname, sc), "Binary",
                            {"operation": orc.BINARY[opname], "scalar": sc}, [SPECIALS]))
    bshapes = [
        ((4, 6, 5, 7), (1, 6, 1, 1)), ((4, 6, 5, 7), (4, 1, 1, 1)), ((4, 6, 5, 7), (1, 1, 1, 7)),
        ((4, 6, 5, 7), (1, 1, 5, 1)), ((4, 6, 5, 7), (1, 6, 5, 7)), ((4, 6, 5, 7), (4, 6, 1, 1)),
        ((4, 1, 5, 7), (1, 6, 1, 7)), ((1, 6, 1, 7), (4, 1, 5, 1)), ((4, 6, 5, 7), (7,)),
        ((5, 7), (4, 6, 5, 7)), ((4, 6, 5, 7), (1,)), ((1,), (3, 2)), ((2, 3, 4, 5, 6), (1, 3, 1, 5, 1)),
        ((2, 1, 3, 1, 2, 1, 3, 1), (1, 2, 1, 3, 1, 2, 1, 3)), ((33, 1), (1, 129)), ((8, 1, 64), (1, 3, 64)),
        ((2, 3, 36), (2, 1, 36)), ((6, 1, 1), (1, 1, 9)),
    ]
    for i, (s1, s2) in enumerate(bshapes):
        for opname in ("Add", "Mul", "Max", "Sub"):
            cs.append(_case("binary_bcast%02d_%s" % (i, opname), "Binary", {"operation": orc.BINARY[opname]},
                            [uniform(400 + i, s1), normal(500 + i, s2)]))
    big_a, big_b = uniform(450, (2, 1, 512, 256)), normal(451, (1, 3, 1, 256))
    for opname in ("Mul", "Sub"):
        cs.append(_case("binary_bcast_reuse_a_%s" % opname, "Binary", {"operation": orc.BINARY[opname]}, [big_a, big_b]))
        cs.append(_case("binary_bcast_reuse_b_%s" % opname, "Binary", {"operation": orc.BINARY[opname]}, [big_b, big_a]))
    # ---- Unary ------------------------------------------------------------------------------
    for opname, code in orc.UNARY.items():
        if opname in ("Sqrt", "Log"):
            x = uniform(600 + code, (1031,), 0.01, 10.0)
        elif opname in ("Asin", "Acos"):
            x = uniform(600 + code, (1031,), -1.0, 1.0)
        else:
            x = uniform(600 + code, (1031,), -10.0, 10.0)
        cs.append(_case("unary_%s" % opname, "Unary", {"operation": code}, [x]))
    for opname in ("Abs", "Square", "Sqrt", "Floor", "Ceil", "Neg", "Reciprocal"):
        cs.append(_case("unary_special_%s" % opname, "Unary", {"operation": orc.UNARY[opname]}, [SPECIALS]))
    for n in (1, 2, 3, 4, 5, 7, 8, 9, 31, 255, 256, 257, 1023, 4099):
        cs.append(_case("unary_ragged_%d" % n, "Unary", {"operation": orc.UNARY["Neg"]}, [uniform(700 + n, (n,))]))
    # ---- Activate ---------------------------------------------------------------------------
    for opname, code in orc.ACTIVATE.items():
        x = normal(800 + code, (2, 6, 5, 9), 0.0, 2.0)
        if opname == "PRelu":
            cs.append(_case("activate_prelu_chan", "Activate", {"type": 0}, [x, normal(850, (6,))]))
            cs.append(_case("activate_prelu_shared", "Activate", {"type": 0}, [x, normal(851, (1,))]))
            cs.append(_case("activate_prelu_2d", "Activate", {"type": 0},
                            [normal(852, (7, 5)), normal(853, (5,))]))
        else:
            cs.append(_case("activate_%s" % opname, "Activate", {"type": code, "slope": float(np.float32(0.1))}, [x]))
    for opname in ("Relu", "Leaky", "Relu6", "HardSwish"):
        cs.append(_case("activate_special_%s" % opname, "Activate",
                        {"type": orc.ACTIVATE[opname], "slope": float(np.float32(0.25))}, [SPECIALS]))
    # ---- Scale ------------------------------------------------------------------------------
    x = normal(900, (3, 8, 5, 7))
    g, bt = normal(901, (8,), 1.0, 0.1), normal(902, (8,), 0.0, 0.1)
    cs.append(_case("scale_blob_sb", "Scale", {"axis": 1, "has_scale": True, "has_bias": True}, [x, g, bt]))
    cs.append(_case("scale_blob_s", "Scale", {"axis": 1, "has_scale": True}, [x, g]))
    cs.append(_case("scale_blob_b", "Scale", {"axis": 1, "has_bias": True}, [x, bt]))
    cs.append(_case("scale_blob_2axes", "Scale", {"axis": 1, "has_scale": True, "has_bias": True},
                    [x, normal(903, (8, 5)), normal(904, (8, 5))]))
    cs.append(_case("scale_blob_axis0", "Scale", {"axis": 0, "has_scale": True, "has_bias": True},
                    [x, normal(905, (3,)), normal(906, (3,))]))
    cs.append(_case("scale_blob_last", "Scale", {"axis": 3, "has_scale": True, "has_bias": True},
                    [x, normal(907, (7,)), normal(908, (7,))]))
    cs.append(_case("scale_value_sb", "Scale", {"axis": 1, "scale_value": [float(v) for v in g],
                                                 "bias_value": [float(v) for v in bt]}, [x]))
    cs.append(_case("scale_value_s1", "Scale", {"axis": 1, "scale_value": [1.5]}, [x]))
    cs.append(_case("scale_value_b1", "Scale", {"axis": 2, "bias_value": [-0.25]}, [x]))
    # the unfused multiply-add known answer: 0.3333333f*0.1f + (-0.033333331f) == +0 exactly
    cs.append(_case("scale_unfused_kat", "Scale", {"axis": 1, "has_scale": True, "has_bias": True},
                    [np.full((1, 1, 1, 4), 0.3333333, np.float32), np.array([0.1], np.float32),
                     np.array([-0.033333331], np.float32)]))
    # ---- Reduce -----------------------------------------------------------------------------
    xr = normal(1000, (4, 6, 5, 7))
    xp = uniform(1001, (4, 6, 5, 7), 0.9, 1.1)
    axes_sets = [[2, 3], [1], [0, 2, 3], [0], [3], [0, 1, 2, 3], [], [1, 2], [0, 3], [1, 3], [0, 1], [0, 2]]
    for opname, code in orc.REDUCE.items():
        for ai, axes in enumerate(axes_sets):
            for keep in (True, False):
                cs.append(_case("reduce_%s_ax%d_k%d" % (opname, ai, int(keep)), "Reduce",
                                {"operation": code, "axes": axes, "keep_dims": keep},
                                [xp if opname == "Prod" else xr]))
    cs.append(_case("reduce_long_row", "Reduce", {"operation": 1, "axes": [1], "keep_dims": True}, [normal(1002, (3, 5000))]))
    cs.append(_case("reduce_long_col", "Reduce", {"operation": 1, "axes": [0], "keep_dims": True}, [normal(1003, (3000, 5))]))
    cs.append(_case("reduce_1d_all", "Reduce", {"operation": 4, "axes": [], "keep_dims": False}, [normal(1004, (10007,))]))
    cs.append(_case("reduce_unsorted_axes", "Reduce", {"operation": 1, "axes": [3, 1], "keep_dims": True}, [xr]))
    nanrow = normal(1005, (4, 33))
    nanrow[1, 5] = np.nan
    nanrow[2, :] = -np.inf
    cs.append(_case("reduce_max_nan", "Reduce", {"operation": 2, "axes": [1], "keep_dims": True}, [nanrow]))
    cs.append(_case("reduce_min_nan", "Reduce", {"operation": 3, "axes": [1], "keep_dims": True}, [nanrow]))
    # extremum is a zero present with both signs, in different lanes / rows / blocks of the kernels
    zs = -np.abs(normal(1008, (6, 40, 9)))
    zs[:, 3, :] = 0.0
    zs[:, 17, ::2] = -0.0
    zs[:, 1, 1::2] = -0.0
    zs[2, :, :] = -0.0
    zs[2, 30, :] = 0.0
    for axes_i, axes in enumerate(([1], [2], [1, 2], [0], [])):
        cs.append(_case("reduce_signed_zero_max_ax%d" % axes_i, "Reduce", {"operation": 2, "axes": axes, "keep_dims": True}, [zs]))
        cs.append(_case("reduce_signed_zero_min_ax%d" % axes_i, "Reduce", {"operation": 3, "axes": axes, "keep_dims": True}, [-zs]))
    # inner-kept reductions with enough planes for the 128-bit fixed-column walk (ragged and 4-aligned K1)
    xc = normal(1009, (900, 64, 7, 7))
    for opname, code in (("Sum", 1), ("Max", 2), ("Avg", 4), ("L2", 6)):
        cs.append(_case("reduce_colwalk_%s" % opname, "Reduce", {"operation": code, "axes": [1], "keep_dims": True}, [xc]))
    cs.append(_case("reduce_colwalk_Prod", "Reduce", {"operation": 0, "axes": [1], "keep_dims": False},
                    [uniform(1010, (900, 64, 7, 7), 0.9, 1.1)]))
    cs.append(_case("reduce_colwalk_tiled_Min", "Reduce", {"operation": 3, "axes": [1], "keep_dims": True}, [normal(1011, (300, 5, 4400))]))
    cs.append(_case("reduce_colwalk_even_Sum", "Reduce", {"operation": 1, "axes": [1], "keep_dims": True}, [normal(1012, (5400, 6, 30))]))
    cs.append(_case("reduce_rows_vec", "Reduce", {"operation": 1, "axes": [2, 3], "keep_dims": True}, [normal(1006, (37, 5, 8, 7))]))
    cs.append(_case("reduce_rows_vec_max", "Reduce", {"operation": 2, "axes": [2, 3], "keep_dims": False}, [normal(1006, (37, 5, 8, 7))]))
    cs.append(_case("reduce_rows_many", "Reduce", {"operation": 4, "axes": [1], "keep_dims": True}, [normal(1007, (3000, 12))]))
    cs.append(_case("reduce_rows_256", "Reduce", {"operation": 6, "axes": [1], "keep_dims": True}, [normal(1008, (19, 1024))]))
    cs.append(_case("reduce_rows_warp", "Reduce", {"operation": 1, "axes": [1], "keep_dims": True}, [normal(1009, (19, 1500))]))
    cs.append(_case("reduce_rkr_small", "Reduce", {"operation": 1, "axes": [0, 2], "keep_dims": True}, [normal(1010, (5, 7, 12))]))
    cs.append(_case("reduce_krk_vec", "Reduce", {"operation": 5, "axes": [1], "keep_dims": True}, [normal(1011, (6, 300, 40))]))
    cs.append(_case("reduce_deep", "Reduce", {"operation": 1, "axes": [1, 3], "keep_dims": False}, [normal(1012, (3, 4, 5, 6, 7))]))
    cs.append(_case("reduce_one_elem", "Reduce", {"operation": 6, "axes": [], "keep_dims": True}, [np.array([[-3.0]], np.float32)]))
    # ---- Eltwise / Axpy ---------------------------------------------------------------------
    e3 = [normal(1200 + k, (3, 5, 7, 9)) for k in range(3)]
    for code, nm in enumerate(("Prod", "Sum", "Max", "Min")):
        cs.append(_case("eltwise_%s_3" % nm, "Eltwise", {"operation": code}, e3))
        cs.append(_case("eltwise_%s_2" % nm, "Eltwise", {"operation": code}, e3[:2]))
    cs.append(_case("eltwise_Sum_coeff", "Eltwise", {"operation": 1, "coeff": [0.5, -1.25, 2.0]}, e3))
    e11 = [normal(1210 + k, (2, 1031)) for k in range(11)]       # more than 8 inputs: chained launches, ragged size
    cs.append(_case("eltwise_Sum_11", "Eltwise", {"operation": 1, "coeff": [float(np.float32(0.1 * (k + 1))) for k in range(11)]}, e11))
    cs.append(_case("eltwise_Max_11", "Eltwise", {"operation": 2}, e11))
    cs.append(_case("eltwise_Prod_9", "Eltwise", {"operation": 0}, [uniform(1230 + k, (4, 64), 0.8, 1.2) for k in range(9)]))
    sp_a, sp_b = special_pairs()
    cs.append(_case("eltwise_Max_special", "Eltwise", {"operation": 2}, [sp_a, sp_b, sp_b]))
    cs.append(_case("eltwise_Sum_special", "Eltwise", {"operation": 1}, [sp_a, sp_b]))
    cs.append(_case("axpy_4d", "Axpy", {}, [normal(1240, (3, 6)), normal(1241, (3, 6, 5, 8)), normal(1242, (3, 6, 5, 8))]))
    cs.append(_case("axpy_alpha4d", "Axpy", {}, [normal(1243, (2, 5, 1, 1)), normal(1244, (2, 5, 7, 7)), normal(1245, (2, 5, 7, 7))]))
    cs.append(_case("axpy_inner3", "Axpy", {}, [normal(1246, (4, 9)), normal(1247, (4, 9, 3)), normal(1248, (4, 9, 3))]))
    xb = normal(1250, (3, 6, 5, 7))
    mean, var = normal(1251, (6,)), uniform(1252, (6,), 0.1, 2.0)
    cs.append(_case("batch_norm_3in", "BatchNorm", {"eps": float(np.float32(1e-5))}, [xb, mean, var]))
    cs.append(_case("batch_norm_scale", "BatchNorm", {}, [xb, mean, var, np.array([0.999], np.float32)]))
    cs.append(_case("batch_norm_scale0", "BatchNorm", {}, [xb, mean, var, np.array([0.0], np.float32)]))
    cs.append(_case("batch_norm_negvar_2d", "BatchNorm", {"eps": float(np.float32(1e-3))},
                    [normal(1253, (9, 4)), normal(1254, (4,)), normal(1255, (4,))]))
    for pn, pv in (("l2", 2.0), ("l1", 1.0), ("l3", 3.0), ("l1_5", 1.5)):
        cs.append(_case("normalize_%s_channels" % pn, "Normalize", {"p": pv, "axis": 1}, [normal(1260, (3, 20, 5, 7))]))
        cs.append(_case("normalize_%s_rows" % pn, "Normalize", {"p": pv, "axis": -1}, [normal(1261, (9, 130))]))
    xz = normal(1262, (4, 6, 3))
    xz[1] = 0.0                                     # all-zero vectors divide by eps
    xz[2, :, 1] = 0.0
    cs.append(_case("normalize_zero_vectors", "Normalize", {"p": 2.0, "axis": 1, "eps": 1e-12}, [xz]))
    cs.append(_case("normalize_big_eps", "Normalize", {"p": 2.0, "axis": 1, "eps": 5.0}, [normal(1263, (4, 6, 3))]))
    cs.append(_case("normalize_axis0_wide", "Normalize", {"p": 2.0, "axis": 0}, [normal(1264, (33, 300))]))
    cs.append(_case("normalize_extremes", "Normalize", {"p": 2.0, "axis": 1},
                    [np.array([[1e-30, 3e-25, -0.0, 0.0], [1e19, -3e18, 2.0, 1e-44], [4.0, 3.0, 0.0, -0.0]], np.float32)]))
    cs.append(_case("normalize_colwalk_tiled", "Normalize", {"p": 2.0, "axis": 1}, [normal(1266, (2, 40, 4400))]))
    cs.append(_case("normalize_colwalk_ragged15_l1", "Normalize", {"p": 1.0, "axis": 1}, [normal(1267, (3, 16, 3, 5))]))
    cs.append(_case("normalize_colwalk_p3", "Normalize", {"p": 3.0, "axis": 1}, [normal(1268, (2, 24, 7, 7))]))
    cs.append(_case("normalize_rows_vec_short", "Normalize", {"p": 2.0, "axis": 1}, [normal(1269, (9, 132))]))
    cs.append(_case("normalize_rows_vec_4096", "Normalize", {"p": 2.0, "axis": 1}, [normal(1270, (5, 4096))]))
    cs.append(_case("normalize_rows_vec_20000_l1", "Normalize", {"p": 1.0, "axis": 1}, [normal(1271, (3, 20000))]))
    cs.append(_case("normalize_rows_too_long", "Normalize", {"p": 2.0, "axis": 1}, [normal(1272, (2, 40000))]))
    cs.append(_case("normalize_long_axis", "Normalize", {"p": 2.0, "axis": 1}, [normal(1265, (2, 5000, 3))]))
    # ---- shape and data-movement operators (bit-exact byte movement) --------------------------
    xm = normal(1300, (2, 6, 5, 4))
    cs.append(_case("reshape_infer", "Reshape", {"shape": [0, -1, 10]}, [xm]))
    cs.append(_case("reshape_sub_range", "Reshape", {"axis": 1, "num_axes": 2, "shape": [3, 10]}, [xm]))
    cs.append(_case("flatten_default", "Flatten", {}, [xm]))
    cs.append(_case("flatten_range", "Flatten", {"axis": 0, "end_axis": 1}, [xm]))
    cs.append(_case("squeeze_all", "Squeeze", {}, [normal(1301, (1, 3, 1, 5))]))
    cs.append(_case("squeeze_listed", "Squeeze", {"axes": [2]}, [normal(1301, (1, 3, 1, 5))]))
    cs.append(_case("unsqueeze", "Unsqueeze", {"axes": [0, -1]}, [normal(1302, (3, 5))]))
    cs.append(_case("concat_axis1", "Concat", {"axis": 1}, [xm, normal(1303, (2, 1, 5, 4)), normal(1304, (2, 9, 5, 4))]))
    cs.append(_case("concat_last_axis_narrow", "Concat", {"axis": -1}, [normal(1305, (7, 3, 4)), normal(1306, (7, 3, 2))]))
    cs.append(_case("concat_axis0_wide", "Concat", {"axis": 0}, [normal(1307, (3, 700)), normal(1308, (2, 700))]))
    cs.append(_case("concat_wide_unaligned", "Concat", {"axis": 1}, [normal(1309, (3, 601)), normal(1310, (3, 515))]))
    cs.append(_case("concat_20_inputs", "Concat", {"axis": 1}, [normal(1320 + k, (2, 1 + k % 3, 3)) for k in range(20)]))
    cs.append(_case("stack_axis0", "Stack", {"axis": 0}, [normal(1340, (4, 5)), normal(1341, (4, 5)), normal(1342, (4, 5))]))
    cs.append(_case("stack_last", "Stack", {"axis": -1}, [normal(1343, (4, 5)), normal(1344, (4, 5))]))
    cs.append(_case("stack_mid_wide", "Stack", {"axis": 1}, [normal(1345, (2, 3, 256)), normal(1346, (2, 3, 256))]))
    cs.append(_case("slice_even", "Slice", {"axis": 1}, [xm], n_tops=3))
    cs.append(_case("slice_points", "Slice", {"axis": 2, "slice_point": [1, 4]}, [xm], n_tops=3))
    cs.append(_case("slice_axis0_wide", "Slice", {"axis": 0, "slice_point": [2]}, [normal(1347, (5, 800))], n_tops=2))
    cs.append(_case("permute_nchw_nhwc", "Permute", {"order": [0, 2, 3, 1]}, [normal(1350, (2, 37, 5, 9))]))
    cs.append(_case("permute_nhwc_nchw", "Permute", {"order": [0, 3, 1, 2]}, [normal(1351, (2, 5, 9, 37))]))
    cs.append(_case("permute_transpose_2d", "Permute", {"order": [1, 0]}, [normal(1352, (70, 33))]))
    cs.append(_case("permute_general", "Permute", {"order": [2, 0, 3, 1]}, [normal(1353, (3, 4, 5, 6))]))
    cs.append(_case("permute_identity", "Permute", {"order": [0, 1, 2]}, [normal(1354, (3, 4, 5))]))
    cs.append(_case("permute_unit_dims", "Permute", {"order": [1, 0, 3, 2]}, [normal(1355, (1, 8, 1, 6))]))
    cs.append(_case("permute_5d", "Permute", {"order": [4, 1, 0, 3, 2]}, [normal(1356, (2, 3, 4, 5, 6))]))
    cs.append(_case("gather_axis0", "Gather", {"axis": 0, "indexes": [3, 0, 0, 2]}, [normal(1360, (5, 7))]))
    cs.append(_case("gather_axis1", "Gather", {"axis": 1, "indexes": [5, 1]}, [xm]))
    cs.append(_case("gather_last", "Gather", {"axis": -1, "indexes": [3, 3, 0]}, [xm]))
    cs.append(_case("pad_grow", "Pad", {"paddings": [1, 2, 3, 0], "value": 2.5}, [xm]))
    cs.append(_case("pad_zero_value_default", "Pad", {"paddings": [0, 0, 2, 2]}, [xm]))
    cs.append(_case("pad_crop", "Pad", {"paddings": [-1, -2, -1, 0]}, [xm]))
    cs.append(_case("pad_mixed", "Pad", {"paddings": [2, -1, -2, 3], "value": -1.0}, [xm]))
    cs.append(_case("pad_none", "Pad", {"paddings": [0, 0, 0, 0]}, [xm]))
    xq = normal(1370, (2, 3, 9, 11))
    cs.append(_case("pool_max_3x3_s2", "Pooling", {"pool": 0, "kernel_size": [3], "stride": [2]}, [xq]))
    cs.append(_case("pool_avg_3x3_s2_pad1", "Pooling", {"pool": 1, "kernel_size": [3], "stride": [2], "pad": [1]}, [xq]))
    cs.append(_case("pool_avg_2x3_floor", "Pooling", {"pool": 1, "kernel_size": [2, 3], "stride": [2, 1], "full_pooling": False}, [xq]))
    cs.append(_case("pool_max_pad_neg_values", "Pooling", {"pool": 0, "kernel_size": [2], "stride": [2], "pad": [1]},
                    [uniform(1371, (2, 3, 6, 6), -5.0, -1.0)]))
    cs.append(_case("pool_global_avg_7x7", "Pooling", {"pool": 1, "global_pooling": True}, [normal(1372, (3, 8, 7, 7))]))
    cs.append(_case("pool_global_max", "Pooling", {"pool": 0, "global_pooling": True}, [normal(1373, (2, 4, 13, 17))]))
    cs.append(_case("pool_global_avg_large", "Pooling", {"pool": 1, "global_pooling": True}, [normal(1374, (2, 4, 13, 17), 1.0, 1.0)]))
    cs.append(_case("pool_3d_max", "Pooling", {"pool": 0, "kernel_size": [2, 3, 2], "stride": [1, 2, 2]}, [normal(1375, (2, 2, 4, 7, 6))]))
    cs.append(_case("pool_3d_avg_pad", "Pooling", {"pool": 1, "kernel_size": [3], "stride": [2], "pad": [1]}, [normal(1376, (1, 3, 5, 6, 7))]))
    xs = normal(1290, (3, 20, 5, 7))
    cs.append(_case("ssd_normalize_defaults", "SSDNormalize", {}, [xs]))
    cs.append(_case("ssd_normalize_across_shared", "SSDNormalize", {"across_spatial": True, "channel_shared": True},
                    [xs, np.array([20.0], np.float32)]))
    cs.append(_case("ssd_normalize_across_channel", "SSDNormalize", {"across_spatial": True, "channel_shared": False},
                    [xs, uniform(1291, (20,), 0.5, 25.0)]))
    cs.append(_case("ssd_normalize_position_channel", "SSDNormalize", {"across_spatial": False, "channel_shared": False,
                                                                         "eps": float(np.float32(1e-10))},
                    [xs, uniform(1292, (20,), 0.5, 25.0)]))
    cs.append(_case("ssd_normalize_position_shared", "SSDNormalize", {"across_spatial": False, "channel_shared": True},
                    [xs, np.array([0.5], np.float32)]))
    cs.append(_case("ssd_normalize_position_noscale", "SSDNormalize", {"across_spatial": False}, [normal(1293, (2, 300, 38))]))
    cs.append(_case("ssd_normalize_position_channel_tiled", "SSDNormalize", {"across_spatial": False, "channel_shared": False},
                    [normal(1294, (2, 24, 4400)), uniform(1295, (24,), 0.5, 25.0)]))
    cs.append(_case("ssd_normalize_position_channel_even", "SSDNormalize", {"across_spatial": False, "channel_shared": False},
                    [normal(1296, (3, 10, 6)), uniform(1297, (10,), 0.5, 25.0)]))
    cs.append(_case("ssd_normalize_position_spatial1", "SSDNormalize", {"across_spatial": False, "channel_shared": False},
                    [normal(1298, (5, 64, 1, 1)), uniform(1299, (64,), 0.5, 25.0)]))
    cs.append(_case("ssd_normalize_across_channel_long", "SSDNormalize", {"across_spatial": True, "channel_shared": False},
                    [normal(1300, (2, 16, 30, 40)), uniform(1301, (16,), 0.5, 25.0)]))
    xg = normal(1270, (3, 12, 5, 7), 0.5, 2.0)
    gs, gb = normal(1271, (12,), 1.0, 0.2), normal(1272, (12,), 0.0, 0.2)
    cs.append(_case("group_norm_g1", "GroupNorm", {"group": 1}, [xg]))
    cs.append(_case("group_norm_g4_affine", "GroupNorm", {"group": 4, "eps": float(np.float32(1e-3))}, [xg, gs, gb]))
    cs.append(_case("group_norm_g12", "GroupNorm", {"group": 12}, [xg]))
    cs.append(_case("group_norm_vec_rows", "GroupNorm", {"group": 2}, [normal(1273, (2, 8, 4, 4)), normal(1274, (8,)), normal(1275, (8,))]))
    cs.append(_case("group_norm_long_rows_affine", "GroupNorm", {"group": 1},
                    [normal(1283, (2, 8, 36, 36), 0.2, 1.0), normal(1284, (8,), 1.0, 0.3), normal(1285, (8,))]))
    cs.append(_case("instance_norm", "InstanceNorm", {}, [xg]))
    cs.append(_case("instance_norm_affine", "InstanceNorm", {}, [xg, gs, gb]))
    xl = normal(1276, (4, 9, 130), -1.0, 3.0)
    cs.append(_case("layer_norm_last", "LayerNorm", {"normalized_shape": [130]}, [xl]))
    cs.append(_case("layer_norm_last_affine", "LayerNorm", {"normalized_shape": [130]}, [xl, normal(1277, (130,)), normal(1278, (130,))]))
    cs.append(_case("layer_norm_two_dims", "LayerNorm", {"normalized_shape": [9, 130], "eps": float(np.float32(1e-6))},
                    [xl, normal(1279, (9, 130)), normal(1280, (9, 130))]))
    cs.append(_case("layer_norm_wide_row", "LayerNorm", {"normalized_shape": [4096]}, [normal(1281, (3, 4096))]))
    cs.append(_case("layer_norm_long_row", "LayerNorm", {"normalized_shape": [40000]}, [normal(1282, (2, 40000), 2.0, 1.0)]))
    cs.append(_case("layer_norm_constant_rows", "LayerNorm", {"normalized_shape": [16]},
                    [np.tile(np.array([[3.5], [0.0], [-2.25]], np.float32), (1, 16))]))
    # ---- Softmax ----------------------------------------------------------------------------
    cs.append(_case("softmax_rows", "Softmax", {"axis": 1}, [normal(1100, (37, 129), 0.0, 3.0)]))
    cs.append(_case("softmax_rows_neg_axis", "Softmax", {"axis": -1}, [normal(1101, (5, 3, 64), 0.0, 3.0)]))
    cs.append(_case("softmax_strided", "Softmax", {"axis": 1}, [normal(1102, (3, 50, 7, 7))]))
    cs.append(_case("softmax_axis0", "Softmax", {"axis": 0}, [normal(1103, (19, 23))]))
    cs.append(_case("softmax_mid", "Softmax", {"axis": 2}, [normal(1104, (2, 3, 11, 5))]))
    cs.append(_case("softmax_dim1", "Softmax", {"axis": 1}, [normal(1105, (7, 1, 3))]))
    cs.append(_case("softmax_long_row", "Softmax", {"axis": 1}, [normal(1106, (2, 20011), 0.0, 3.0)]))
    cs.append(_case("softmax_cluster8", "Softmax", {"axis": 1}, [normal(1108, (2, 1000, 7, 7))]))
    cs.append(_case("softmax_cluster2", "Softmax", {"axis": 1}, [normal(1109, (3, 300, 49))]))
    cs.append(_case("softmax_cluster4_wide", "Softmax", {"axis": 1}, [normal(1110, (2, 100, 300))]))
    cs.append(_case("softmax_plane_two_pass", "Softmax", {"axis": 1}, [normal(1111, (2, 300, 300), 0.0, 3.0)]))
    cs.append(_case("softmax_inner2", "Softmax", {"axis": 0}, [normal(1112, (700, 2))]))
    # strided-softmax block geometries: several tiny planes packed into one block (odd and 4-aligned
    # plane sizes), inner extents above one column tile (256) with and without a ragged last tile,
    # a [900, 52] plane (512-thread blocks), and a long channel axis with a narrow inner extent
    cs.append(_case("softmax_patch_packed_odd", "Softmax", {"axis": 1}, [normal(1113, (11, 7, 3, 3))]))
    cs.append(_case("softmax_patch_packed_vec", "Softmax", {"axis": 1}, [normal(1114, (13, 8, 10))]))
    cs.append(_case("softmax_patch_tiles_vec", "Softmax", {"axis": 1}, [normal(1115, (2, 21, 520), 0.0, 3.0)]))
    cs.append(_case("softmax_patch_tiles_scalar", "Softmax", {"axis": 1}, [normal(1116, (2, 5, 301))]))
    cs.append(_case("softmax_patch_big", "Softmax", {"axis": 1}, [normal(1117, (2, 900, 52))]))
    cs.append(_case("softmax_patch_too_tall", "Softmax", {"axis": 1}, [normal(1118, (1, 7000, 12))]))
    # the 128-bit fixed-column walk: column tiles of long rows, ragged inner = 15, packed tiny planes
    cs.append(_case("softmax_colwalk_tiled", "Softmax", {"axis": 1}, [normal(1119, (2, 9, 4400), 0.0, 3.0)]))
    cs.append(_case("softmax_colwalk_ragged15", "Softmax", {"axis": 1}, [normal(1120, (5, 12, 3, 5))]))
    cs.append(_case("softmax_colwalk_partial_batch", "Softmax", {"axis": 1}, [normal(1121, (3, 1004, 7, 7))]))
    # a NaN poisons its whole column (every output is divided by the NaN sum) and nothing else
    xn = normal(1122, (2, 8, 6))
    xn[1, 3, 4] = np.nan
    cs.append(_case("softmax_nan_column", "Softmax", {"axis": 1}, [xn]))
    xn2 = normal(1123, (3, 40))
    xn2[2, 7] = np.nan
    cs.append(_case("softmax_nan_row", "Softmax", {"axis": 1}, [xn2]))
    cs.append(_case("softmax_huge_logits", "Softmax", {"axis": 1}, [normal(1107, (4, 300), 0.0, 200.0)]))
    return cs


def _shape_op(op, a, shape):
    """Output shape of the zero-copy operators (Reshape / Flatten / Squeeze / Unsqueeze)."""
    shape = list(shape)
    n = len(shape)
    if op == "Reshape":
        start = a.get("axis", 0) % n
        end = n if a.get("num_axes", -1) == -1 else start + a["num_axes"]
        new = [shape[start + k] if d == 0 else d for k, d in enumerate(a["shape"])]
        out = shape[:start] + new + shape[end:]
        if -1 in out:
            known = int(np.prod([d for d in out if d != -1], dtype=np.int64))
            out[out.index(-1)] = int(np.prod(shape, dtype=np.int64)) // known
        return out
    if op == "Flatten":
        ax, end = a.get("axis", 1), a.get("end_axis", -1)
        end = n - 1 if end == -1 else end
        return shape[:ax] + [int(np.prod(shape[ax:end + 1], dtype=np.int64))] + shape[end + 1:]
    if op == "Squeeze":
        axes = a.get("axes", [])
        return [d for k, d in enumerate(shape) if (d > 1 if not axes else k not in axes)]
    axes = [ax + n + 1 if ax < 0 else ax for ax in a["axes"]]
    out, it = [], iter(shape)
    for k in range(n + len(axes)):
        out.append(1 if k in axes else next(it))
    return out


def _slice_sizes(a, extent, n_tops):
    pts = a.get("slice_point", [])
    if not pts:
        return [extent // n_tops] * n_tops
    edges = [0] + list(pts) + [extent]
    return [edges[k + 1] - edges[k] for k in range(n_tops)]


def _movement(case, impl, back):
    """Shape / data-movement cases on `impl` (the oracle module or shadow_b200.functional); `back`
    turns a result into a numpy array.  None when the case is not one of these operators."""
    op, a, x = case["op"], dict(case["args"]), case["_args_inputs"] if "_args_inputs" in case else case["inputs"]
    if op in ("Reshape", "Flatten", "Squeeze", "Unsqueeze"):
        return back(x[0]).reshape(_shape_op(op, a, case["inputs"][0].shape))
    if op == "Concat":
        return back(impl.concat(x, a.get("axis", 1)))
    if op == "Stack":
        return back(impl.stack(x, a.get("axis", 0)))
    if op == "Slice":
        axis = a.get("axis", 1) % case["inputs"][0].ndim
        outs = impl.slice_(x[0], axis, _slice_sizes(a, case["inputs"][0].shape[axis], case["n_tops"]))
        return np.concatenate([back(o).ravel() for o in outs])
    if op == "Permute":
        return back(impl.permute(x[0], a["order"]))
    if op == "Pad":
        return back(impl.pad(x[0], a["paddings"], a.get("value", 0.0)))
    return None


def run_port(case) -> np.ndarray:
    """Evaluate a case with the C restatement + Python front-end rules."""
    op, a, x = case["op"], dict(case["args"]), case["inputs"]
    if op == "Binary":
        if "scalar" in a:
            return orc.binary_scalar(x[0], a["scalar"], a["operation"])
        return orc.binary(x[0], x[1], a["operation"])
    if op == "Unary":
        return orc.unary(x[0], a["operation"])
    if op == "Activate":
        t = a.get("type", 1)
        return orc.activate(x[0], t, a.get("slope", 0.1), x[1] if t == 0 else None)
    if op == "Scale":
        axis = a.get("axis", 1)
        hs, hb = a.get("has_scale", False), a.get("has_bias", False)
        if hs and hb:
            return orc.scale(x[0], axis, x[1], x[2])
        if hs:
            return orc.scale(x[0], axis, x[1], None)
        if hb:
            return orc.scale(x[0], axis, None, x[1])
        dim = x[0].shape[axis]
        sv, bv = list(a.get("scale_value", [])), list(a.get("bias_value", []))
        sv = sv * dim if len(sv) == 1 else sv
        bv = bv * dim if len(bv) == 1 else bv
        return orc.scale(x[0], axis, np.array(sv, np.float32) if sv else None,
                         np.array(bv, np.float32) if bv else None)
    if op == "Reduce":
        return orc.reduce(x[0], a.get("operation", 0), a.get("axes", []), a.get("keep_dims", True))
    if op == "Softmax":
        return orc.softmax(x[0], a.get("axis", 1))
    if op == "Eltwise":
        return orc.eltwise(x, a["operation"], a.get("coeff", []))
    if op == "Axpy":
        return orc.axpy(x[0], x[1], x[2])
    mv = _movement(case, orc, lambda v: v)
    if mv is not None:
        return mv
    if op == "SSDNormalize":
        return orc.ssd_normalize(x[0], x[1] if len(x) == 2 else None, a.get("across_spatial", True),
                                 a.get("channel_shared", True), a.get("eps", 1e-5))
    if op == "GroupNorm":
        return orc.group_norm(x[0], a.get("group", 1), x[1] if len(x) == 3 else None, x[2] if len(x) == 3 else None,
                              a.get("eps", 1e-5))
    if op == "InstanceNorm":
        return orc.group_norm(x[0], x[0].shape[1], x[1] if len(x) == 3 else None, x[2] if len(x) == 3 else None,
                              a.get("eps", 1e-5))
    if op == "LayerNorm":
        return orc.layer_norm(x[0], a["normalized_shape"], x[1] if len(x) == 3 else None, x[2] if len(x) == 3 else None,
                              a.get("eps", 1e-5))
    if op == "Gather":
        return orc.gather(x[0], a["indexes"], a.get("axis", 0))
    if op == "Pooling":
        return orc.pooling(x[0], a.get("pool", 0), a.get("kernel_size", []), a.get("stride", [1]), a.get("pad", [0]),
                           a.get("global_pooling", False), a.get("full_pooling", True))
    if op == "Normalize":
        return orc.normalize(x[0], a.get("axis", 1), a.get("p", 2.0), a.get("eps", 1e-12))
    if op == "BatchNorm":
        return orc.batch_norm(x[0], x[1], x[2], x[3] if len(x) == 4 else None, a.get("eps", 1e-5))
    raise KeyError(op)


def run_net(library, case, backend="Native", device_id=0):
    """Evaluate a case through the Network API of `library` (reference build or product)."""
    from shadow_b200.netapi import Net
    names = ["in%d" % i for i in range(len(case["inputs"]))]
    net = Net(library, case["name"])
    net.input({n: (x.shape if x.ndim else (1,)) for n, x in zip(names, case["inputs"])})
    n_tops = case.get("n_tops", 1)
    if n_tops == 1:
        net.op(case["op"], names, ["out"], **case["args"])
        net.load(backend, device_id=device_id, out_blobs=["out"])
        net.forward(dict(zip(names, case["inputs"])))
        return net.blob("out")
    tops = ["out%d" % k for k in range(n_tops)]       # several outputs: returned flattened, one after another
    net.op(case["op"], names, tops, **case["args"])
    net.load(backend, device_id=device_id, out_blobs=tops)
    net.forward(dict(zip(names, case["inputs"])))
    return np.concatenate([net.blob(t).ravel() for t in tops])


def tolerance_class(case) -> str:
    """'exact', 'ulp2' or 'rel' (relative error <= 1e-5*log2(n))."""
    op, a = case["op"], case["args"]
    if op == "Binary":
        return "ulp2" if a["operation"] == 4 else "exact"
    if op == "Unary":
        return "ulp2" if a["operation"] in (3, 4, 5, 6, 7, 8, 9, 10) else "exact"
    if op == "Activate":
        t = a.get("type", 1)
        return "gelu" if t == 8 else ("ulp2" if t in (3, 4, 5) else "exact")
    if op == "Scale":
        return "exact"
    if op == "Reduce":
        if case["name"].startswith("reduce_signed_zero"):
            return "exact_up_to_zero_sign"
        return "exact" if a.get("operation", 0) in (2, 3) else "rel"
    if op in ("Eltwise", "Axpy", "BatchNorm", "Reshape", "Flatten", "Squeeze", "Unsqueeze", "Concat", "Stack", "Slice",
              "Permute", "Gather", "Pad"):
        return "exact"
    if op in ("GroupNorm", "InstanceNorm", "LayerNorm"):
        return "rownorm"
    if op == "Pooling":
        # max, and averages over windows of up to 64 elements (summed in the reference's order), are exact;
        # larger windows are summed by a warp in double
        x = case["inputs"][0]
        window = int(np.prod(x.shape[2:])) if a.get("global_pooling", False) else int(np.prod(
            a["kernel_size"] * (x.ndim - 2) if len(a["kernel_size"]) == 1 else a["kernel_size"]))
        return "exact" if a.get("pool", 0) == 0 or window <= 64 else "rel"
    if op == "SSDNormalize":   # only the order of the double additions differs from the reference
        return "ulp2"
    if op == "Normalize":   # p = 1, 2: only the order of the double additions differs from the reference
        return "ulp2" if a.get("p", 2.0) in (1.0, 2.0) else "rel"
    return "rel"


def run_cuda(case, device="cuda:0"):
    """Evaluate a case through the kernel C ABI (shadow_b200.functional) on device tensors."""
    import torch
    from shadow_b200 import functional as F
    op, a = case["op"], dict(case["args"])
    x = [torch.from_numpy(np.ascontiguousarray(v)).to(device) for v in case["inputs"]]
    if op == "Binary":
        y = F.binary_scalar(x[0], a["scalar"], a["operation"]) if "scalar" in a else F.binary(x[0], x[1], a["operation"])
    elif op == "Unary":
        y = F.unary(x[0], a["operation"])
    elif op == "Activate":
        t = a.get("type", 1)
        y = F.activate(x[0], t, a.get("slope", 0.1), x[1] if t == 0 else None)
    elif op == "Scale":
        axis = a.get("axis", 1)
        hs, hb = a.get("has_scale", False), a.get("has_bias", False)
        if hs and hb:
            y = F.scale(x[0], axis, x[1], x[2])
        elif hs:
            y = F.scale(x[0], axis, x[1], None)
        elif hb:
            y = F.scale(x[0], axis, None, x[1])
        else:
            dim = x[0].shape[axis]
            sv, bv = list(a.get("scale_value", [])), list(a.get("bias_value", []))
            sv = sv * dim if len(sv) == 1 else sv
            bv = bv * dim if len(bv) == 1 else bv
            dev = lambda v: torch.tensor(v, dtype=torch.float32, device=device) if v else None  # noqa: E731
            y = F.scale(x[0], axis, dev(sv), dev(bv))
    elif op == "Reduce":
        y = F.reduce(x[0], a.get("operation", 0), a.get("axes", []), a.get("keep_dims", True))
    elif op == "Softmax":
        y = F.softmax(x[0], a.get("axis", 1))
    elif op == "Eltwise":
        y = F.eltwise(x, a["operation"], a.get("coeff", []))
    elif op == "Axpy":
        y = F.axpy(x[0], x[1], x[2])
    elif op in ("Reshape", "Flatten", "Squeeze", "Unsqueeze", "Concat", "Stack", "Slice", "Permute", "Pad"):
        torch.cuda.synchronize()
        return _movement(dict(case, _args_inputs=x), F, lambda t: t.cpu().numpy())
    elif op == "Pooling":
        y = F.pooling(x[0], a.get("pool", 0), a.get("kernel_size", []), a.get("stride", [1]), a.get("pad", [0]),
                      a.get("global_pooling", False), a.get("full_pooling", True))
    elif op == "Gather":
        y = F.gather(x[0], torch.tensor(a["indexes"], dtype=torch.int32, device=device), a.get("axis", 0))
    elif op == "SSDNormalize":
        y = F.ssd_normalize(x[0], x[1] if len(x) == 2 else None, a.get("across_spatial", True),
                            a.get("channel_shared", True), a.get("eps", 1e-5))
    elif op == "GroupNorm":
        y = F.group_norm(x[0], a.get("group", 1), x[1] if len(x) == 3 else None, x[2] if len(x) == 3 else None,
                         a.get("eps", 1e-5))
    elif op == "InstanceNorm":
        y = F.instance_norm(x[0], x[1] if len(x) == 3 else None, x[2] if len(x) == 3 else None, a.get("eps", 1e-5))
    elif op == "LayerNorm":
        y = F.layer_norm(x[0], a["normalized_shape"], x[1] if len(x) == 3 else None, x[2] if len(x) == 3 else None,
                         a.get("eps", 1e-5))
    elif op == "Normalize":
        y = F.normalize(x[0], a.get("axis", 1), a.get("p", 2.0), a.get("eps", 1e-12))
    elif op == "BatchNorm":
        sf = 1.0
        if len(x) == 4:
            sc = np.float32(case["inputs"][3].ravel()[0])
            sf = float(np.float32(0) if sc == 0 else np.float32(1) / sc)
        y = F.batch_norm(x[0], x[1], x[2], sf, a.get("eps", 1e-5))
    else:
        raise KeyError(op)
    torch.cuda.synchronize()
    return y.cpu().numpy()


def reduced_length(case) -> int:
    x = case["inputs"][0]
    if case["op"] in ("Softmax", "Normalize"):
        return int(x.shape[case["args"].get("axis", 1)])
    if case["op"] == "Pooling":
        return int(np.prod(x.shape[2:]))
    axes = case["args"].get("axes", []) or list(range(x.ndim))
    return int(np.prod([x.shape[a] for a in axes]))


def assert_parity(case, got: np.ndarray, want: np.ndarray):
    """The parity bar: bit-exact / <= 2 ulp / relative error <= 1e-5*log2(n)."""
    assert tuple(got.shape) == tuple(want.shape), (got.shape, want.shape)
    cls = tolerance_class(case)
    if cls == "exact":
        # bit-for-bit, signed zeros included; a NaN matches a NaN whatever its sign/payload bits
        # (x86 produces the negative default NaN for inf-inf, the GPU the positive canonical one)
        gb, wb = got.ravel().view(np.uint32), want.ravel().view(np.uint32)
        bad = (gb != wb) & ~(np.isnan(got.ravel()) & np.isnan(want.ravel()))
        assert not bad.any(), "%s: not bit-exact at %d elements, max ulp %d" % (
            case["name"], int(bad.sum()), int(orc.ulp_distance(got, want).max()))
    elif cls == "exact_up_to_zero_sign":
        # Reduce Max/Min whose extremum is a zero that occurs with both signs: the reference keeps the
        # zero it meets first in its left-to-right loop; the GPU merges lanes and blocks in tree
        # order, so the SIGN of such a zero may differ.  Everything else is bit-for-bit.
        gb, wb = got.ravel().view(np.uint32), want.ravel().view(np.uint32)
        both_zero = (got.ravel() == 0) & (want.ravel() == 0)
        bad = (gb != wb) & ~both_zero & ~(np.isnan(got.ravel()) & np.isnan(want.ravel()))
        assert not bad.any(), "%s: differs beyond the sign of a zero at %d elements" % (case["name"], int(bad.sum()))
    elif cls == "gelu":
        # 0.5f*x*(1+erf(0.707107f*x)): for x << 0 the sum 1+erf cancels, so one ulp of difference in
        # erf (glibc's erff is within 1 ulp of the true value, the GPU's is correctly rounded) is
        # magnified in the result.  Bar: 2 ulp of the result plus one ulp of erf (2^-24) times |0.5x|.
        x = case["inputs"][0].astype(np.float64).ravel()
        g, w = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
        tol = 2 * np.spacing(np.abs(want.ravel()).astype(np.float32)).astype(np.float64) + np.abs(0.5 * x) * 2.0 ** -24
        assert np.all(np.abs(g - w) <= tol), "%s: |err| above 2 ulp + |x/2|*2^-24" % case["name"]
    elif cls == "rownorm":
        # mean and variance are double sums rounded to float; a different order of the additions can
        # move either by one float ulp.  One ulp of the mean shifts every centred value of the row by
        # that much ABSOLUTELY (x - mean cancels), so the bar is absolute per row:
        # 2^-22 * max|x| / sqrt(var + eps) (times |scale|), plus 2^-22 relative.
        x = case["inputs"][0].astype(np.float64)
        a = case["args"]
        if case["op"] == "LayerNorm":
            inner = int(np.prod(a["normalized_shape"]))
        else:
            group = a.get("group", 1) if case["op"] == "GroupNorm" else x.shape[1]
            inner = x.size // (x.shape[0] * group)
        rows = x.reshape(-1, inner)
        sd = np.sqrt(rows.var(axis=1) + a.get("eps", 1e-5))
        row_tol = (2.0 ** -22) * np.abs(rows).max(axis=1) / sd
        tol = np.repeat(row_tol, inner)
        if len(case["inputs"]) == 3:
            sc = np.abs(case["inputs"][1].astype(np.float64)).ravel()
            if case["op"] == "LayerNorm":
                tol = tol * np.tile(sc, x.size // sc.size)
            else:
                spatial = int(np.prod(x.shape[2:]))
                tol = tol * np.tile(np.repeat(sc, spatial), x.shape[0])
        g, w = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
        assert np.all(np.abs(g - w) <= tol + (2.0 ** -22) * np.abs(w)), "%s: max excess %g" % (
            case["name"], float(np.max(np.abs(g - w) - tol - (2.0 ** -22) * np.abs(w))))
    elif cls == "ulp2":
        d = orc.ulp_distance(got, want)
        assert int(d.max()) <= 2, "%s: max ulp %d" % (case["name"], int(d.max()))
    else:
        n = max(reduced_length(case), 2)
        tol = 1e-5 * np.log2(n)
        g, w = got.astype(np.float64).ravel(), want.astype(np.float64).ravel()
        both_nan = np.isnan(g) & np.isnan(w)
        same_inf = np.isinf(g) & np.isinf(w) & (np.sign(g) == np.sign(w))
        ok = both_nan | same_inf
        err = np.abs(g - w)
        denom = np.abs(w)
        # a NaN on one side only (or infinities of different sign) is a failure, not something to skip
        one_sided = (np.isnan(g) ^ np.isnan(w)) | ((np.isinf(g) | np.isinf(w)) & ~ok)
        assert not one_sided.any(), "%s: NaN/inf on one side only at %d elements" % (case["name"], int(one_sided.sum()))
        with np.errstate(invalid="ignore", divide="ignore"):
            rel = np.where(ok, 0.0, np.where(denom > 0, err / np.maximum(denom, 1e-300), err))
        # outputs that are exactly 0 in the reference (underflowed softmax terms) must be ~0 here
        assert float(np.max(rel)) <= tol, "%s: rel err %.3g > %.3g" % (case["name"], float(np.max(rel)), tol)
