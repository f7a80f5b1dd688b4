"""Operation lists of the C-ABI, mirroring the X-macro lists of include/solid_core_gpu.h
(a CPU test preprocesses the header and checks that the two agree)."""

FILL_OPS = {"fill": "all", "fill_nan": "float"}
UNARY_OPS = {
    "negative": "all_nouint", "conj": "complex", "reciprocal": "all_nobool",
    "bitwise_not": "integer_bool", "logical_not": "bool",
    **{n: "all_nobool" for n in ["sin", "cos", "tan", "sinh", "cosh", "tanh", "arcsin", "arccos", "arctan",
                                  "arcsinh", "arccosh", "arctanh", "sqrt", "cbrt", "square", "exp", "exp2",
                                  "exp10", "expm1", "log", "log2", "log10", "log1p"]},
    "fabs": "all", "sign": "all", "ceil": "float", "floor": "float", "trunc": "float", "round": "float",
    "isinf": "all", "isnan": "all", "isfinite": "all", "isposinf": "all_nocomplex", "isneginf": "all_nocomplex",
    "absolute": "all",
}
BINARY_OPS = {
    "add": "all", "subtract": "all", "multiply": "all", "divide": "all", "true_divide": "all",
    "floor_divide": "all_nocomplex", "mod": "all_nocomplex", "fmod": "all_nocomplex",
    "bitwise_and": "integer_bool", "bitwise_or": "integer_bool", "bitwise_xor": "integer_bool",
    "logical_and": "bool", "logical_or": "bool", "logical_xor": "bool",
    "lt": "all", "le": "all", "ge": "all", "gt": "all", "eq": "all", "ne": "all",
    "min": "all", "max": "all", "fmin": "all", "fmax": "all",
    "bitshift_left": "integer_bool", "bitshift_right": "integer_bool", "power": "all",
}
COMPARE_OPS = ["lt", "le", "ge", "gt", "eq", "ne"]
# unary functions fused with their domain test: name -> (type group, reference test)
CHECKED_OPS = {"sqrt": "real", "log": "real", "log2": "real", "log10": "real", "log1p": "real", "arccosh": "real",
               "arcsin": "real", "arccos": "real", "arctanh": "real", "reciprocal": "real"}
GEMM_OPS = {"gemm": "integer_bool", "gemm_with_plan": "integer_bool"}
INDEX_OPS = {"get_index": "all", "set_index": "all", "fill_index": "all", "add_if_negative": "sint",
             "index_to_offset": "integer"}
STEPS_OPS = {"steps_int64": "all", "steps_double": "all", "steps_cdouble": "complex"}
# second operand passed by value (solid_gpu_<op>_scalar_<type>)
SCALAR_OPS = {"add": "all", "subtract": "all", "multiply": "all",
              "bitwise_and": "integer_bool", "bitwise_or": "integer_bool", "bitwise_xor": "integer_bool"}
REDUCE_BOOL_OPS = {"any": "all", "all": "all", "all_finite": "float", "any_inf": "float", "any_nan": "float"}
REDUCE_BOUND1_OPS = {"all_lt": "all", "all_le": "all", "all_gt": "all", "all_ge": "all"}
REDUCE_BOUND2_OPS = {"all_gtlt": "all", "all_gtle": "all", "all_gelt": "all", "all_gele": "all"}
REDUCE_U64_OPS = {"nnz": "all", "nnz_nan": "all"}
REDUCE_VOID_OPS = {n: "all" for n in ["sum", "sum_nan", "prod", "prod_nan", "sum_abs", "sum_abs_nan", "maximum",
                                      "minimum", "maximum_abs", "minimum_abs", "norm2", "norm2_nan"]}
REDUCE_NORM_OPS = {"norm": "all", "norm_nan": "all"}
AXIS_OPS = {("axis_" + n): g for n, g in {**{k: v for k, v in REDUCE_BOOL_OPS.items()},
                                           **REDUCE_U64_OPS, **REDUCE_VOID_OPS}.items()}
AXIS_NORM_OPS = {"axis_norm": "all", "axis_norm_nan": "all"}


def reduce_result_type(op: str, dtype: str) -> str:
    """Element type of the result of a reduction `op` (global or axis_ form) over `dtype`."""
    from . import dtypes as dt
    op = op[5:] if op.startswith("axis_") else op
    if op in REDUCE_BOOL_OPS or op in REDUCE_BOUND1_OPS or op in REDUCE_BOUND2_OPS:
        return "bool"
    if op in REDUCE_U64_OPS:
        return "uint64"
    if op in ("sum", "sum_nan", "prod", "prod_nan"):
        return dt.sum_type(dtype)
    if op in ("sum_abs", "sum_abs_nan"):
        return "uint64" if dtype in dt.GROUPS["integer_bool"] else dt.abs_type(dtype)
    if op in ("maximum", "minimum"):
        return dtype
    if op in ("maximum_abs", "minimum_abs"):
        return dt.abs_type(dtype)
    if op in ("norm", "norm_nan", "norm2", "norm2_nan"):
        return dt.norm_type(dtype)
    raise KeyError(op)
