// Element-wise op kinds, numbered as the reference numbers them
// (crates/tt-kernels/src/kind.rs:12-26 and crates/tt-kernels/src/sfpu/ops.rs:24-251),
// so an `Eltwise{kind,..}` crosses the boundary unchanged.
#pragma once
#include <stdint.h>

// X(name, value, arity)  arity: 1 unary, 2 binary, 3 ternary
#define B200_KINDS(X)                                                                        \
  X(ADD, 1, 2) X(SUB, 2, 2) X(MUL, 3, 2) X(MUL_SCALAR, 4, 1) X(RELU, 5, 1)                  \
  X(RELU_BACKWARD, 6, 2) X(ADD_ROW, 7, 2) X(ADD_SCALAR, 11, 1)                              \
  X(RECIP, 0x100, 1) X(DIV, 0x101, 2) X(DIV_SCALAR, 0x102, 1) X(EXP, 0x103, 1)             \
  X(LOG, 0x104, 1) X(BOOL_NOT, 0x105, 1) X(BOOL_AND, 0x106, 2) X(BOOL_OR, 0x107, 2)        \
  X(BOOL_XOR, 0x108, 2) X(NEG, 0x109, 1) X(ABS, 0x10a, 1) X(SIGN, 0x10b, 1)                \
  X(CLAMP, 0x10c, 1) X(CLAMP_MIN, 0x10d, 1) X(CLAMP_MAX, 0x10e, 1) X(LEAKY_RELU, 0x10f, 1) \
  X(HARD_SIGMOID, 0x110, 1) X(EQ, 0x111, 2) X(NE, 0x112, 2) X(GT, 0x113, 2) X(GE, 0x114, 2) \
  X(LT, 0x115, 2) X(LE, 0x116, 2) X(EQ_S, 0x117, 1) X(NE_S, 0x118, 1) X(GT_S, 0x119, 1)    \
  X(GE_S, 0x11a, 1) X(LT_S, 0x11b, 1) X(LE_S, 0x11c, 1) X(IS_NAN, 0x11d, 1)                \
  X(IS_INF, 0x11e, 1) X(MASK_FILL, 0x11f, 2) X(MASK_WHERE, 0x120, 3) X(PRELU, 0x121, 2)    \
  X(FILL, 0x122, 1) X(SQRT, 0x123, 1) X(RSQRT, 0x124, 1) X(LOG1P, 0x125, 1) X(POW, 0x126, 2) \
  X(POW_S, 0x127, 1) X(POW_I, 0x128, 2) X(I32_TO_F32, 0x129, 1) X(EXPM1, 0x12a, 1)         \
  X(SIGMOID, 0x12b, 1) X(SIGMOID_BACKWARD, 0x12c, 2) X(TANH, 0x12d, 1) X(ERF, 0x12e, 1)    \
  X(GELU, 0x12f, 1) X(GELU_BACKWARD, 0x130, 2) X(SINH, 0x131, 1) X(COSH, 0x132, 1)         \
  X(ASINH, 0x133, 1) X(ACOSH, 0x134, 1) X(ATANH, 0x135, 1) X(LOG_SIGMOID, 0x136, 1)        \
  X(LOG_SIGMOID_BACKWARD, 0x137, 2) X(SIN, 0x138, 1) X(COS, 0x139, 1) X(TAN, 0x13a, 1)     \
  X(ATAN, 0x13b, 1) X(ATAN2, 0x13c, 2) X(ASIN, 0x13d, 1) X(ACOS, 0x13e, 1)                 \
  X(BOOL_TO_F32, 0x13f, 1) X(BOOL_TO_I32, 0x140, 1) X(REM, 0x141, 2) X(REM_S, 0x142, 1)    \
  X(INDEX_TO_I32, 0x160, 1) X(INT_MASK_WHERE, 0x161, 3) X(BOOL_MASK_WHERE, 0x162, 3)       \
  X(INT_MASK_FILL, 0x163, 2) X(BOOL_MASK_FILL, 0x164, 2) X(INT_ABS, 0x165, 1)              \
  X(INT_ADD, 0x170, 2) X(INT_SUB, 0x171, 2) X(INT_MUL, 0x172, 2) X(INT_AND, 0x173, 2)      \
  X(INT_OR, 0x174, 2) X(INT_XOR, 0x175, 2) X(INT_SHL, 0x176, 2) X(INT_SHR, 0x177, 2)       \
  X(INT_EQ, 0x178, 2) X(INT_NE, 0x179, 2) X(INT_GT, 0x17a, 2) X(INT_GE, 0x17b, 2)          \
  X(INT_LT, 0x17c, 2) X(INT_LE, 0x17d, 2) X(INT_NOT, 0x17e, 1) X(INT_ADD_S, 0x180, 1)      \
  X(INT_SUB_S, 0x181, 1) X(INT_MUL_S, 0x182, 1) X(INT_AND_S, 0x183, 1) X(INT_OR_S, 0x184, 1) \
  X(INT_XOR_S, 0x185, 1) X(INT_SHL_S, 0x186, 1) X(INT_SHR_S, 0x187, 1) X(INT_EQ_S, 0x188, 1) \
  X(INT_NE_S, 0x189, 1) X(INT_GT_S, 0x18a, 1) X(INT_GE_S, 0x18b, 1) X(INT_LT_S, 0x18c, 1)  \
  X(INT_LE_S, 0x18d, 1) X(INT_DIV, 0x18e, 2) X(INT_REM, 0x18f, 2) X(ROUND, 0x190, 1)       \
  X(FLOOR, 0x191, 1) X(CEIL, 0x192, 1) X(TRUNC, 0x193, 1) X(F32_TO_I32, 0x194, 1)          \
  X(POW2_FLOOR, 0x195, 1) X(POW2_FLOOR_INV, 0x196, 1) X(INT_DIV_S, 0x1a0, 1)               \
  X(INT_REM_S, 0x1a1, 1) X(ADD_RELU, 0x1f0, 2) X(SILU, 0x1f1, 1) X(SILU_MUL, 0x1f2, 2)     \
  X(SUB_EXP, 0x1f3, 2) X(MUL_ADD, 0x1f4, 3) X(SCALE_MASK_FILL, 0x1f5, 2)                   \
  /* not in the reference: the tanh form of GELU that the benchmark suite names */          \
  X(GELU_TANH, 0x2f0, 1)

namespace kind {
#define B200_KIND_CONST(name, value, arity) constexpr uint32_t name = value;
B200_KINDS(B200_KIND_CONST)
#undef B200_KIND_CONST
inline int arity(uint32_t k) {
  switch (k) {
#define B200_KIND_ARITY(name, value, ar) case value: return ar;
    B200_KINDS(B200_KIND_ARITY)
#undef B200_KIND_ARITY
    default: return 0;
  }
}
inline const char* name(uint32_t k) {
  switch (k) {
#define B200_KIND_NAME(nm, value, ar) case value: return #nm;
    B200_KINDS(B200_KIND_NAME)
#undef B200_KIND_NAME
    default: return "?";
  }
}
// Kinds whose second operand may be a row, a column or repeated whole rows
// (crates/tt-kernels/src/sfpu/ops.rs:2510-2533).
inline bool broadcasts(uint32_t k) {
  switch (k) {
    case ADD: case ADD_ROW: case ADD_RELU: case SUB_EXP: case SUB: case MUL: case DIV:
    case BOOL_AND: case BOOL_OR: case BOOL_XOR:
    case EQ: case NE: case GT: case GE: case LT: case LE:
    case MASK_FILL: case INT_MASK_FILL: case BOOL_MASK_FILL: case SCALE_MASK_FILL: case PRELU:
    case INT_ADD: case INT_SUB: case INT_MUL: case INT_AND: case INT_OR: case INT_XOR:
    case INT_SHL: case INT_SHR: case INT_EQ: case INT_NE: case INT_GT: case INT_GE:
    case INT_LT: case INT_LE: case INT_DIV: case INT_REM:
      return true;
    default: return false;
  }
}
// Result element of a kind: 0 F32, 1 I32, 2 Bool (sfpu/ops.rs:296 `elems`).
inline int result_elem(uint32_t k) {
  if ((k >= EQ && k <= IS_INF) || (k >= BOOL_NOT && k <= BOOL_XOR) || k == BOOL_MASK_WHERE ||
      k == BOOL_MASK_FILL || (k >= INT_EQ && k <= INT_LE) || (k >= INT_EQ_S && k <= INT_LE_S))
    return 2;
  if (k == INDEX_TO_I32 || k == INT_MASK_WHERE || k == INT_MASK_FILL || k == INT_ABS ||
      (k >= INT_ADD && k <= INT_SHR) || k == INT_NOT || (k >= INT_ADD_S && k <= INT_SHR_S) ||
      k == INT_DIV || k == INT_REM || k == INT_DIV_S || k == INT_REM_S || k == F32_TO_I32 ||
      k == BOOL_TO_I32)
    return 1;
  return 0;
}
}  // namespace kind
