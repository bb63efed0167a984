// Argument checks shared by the extern "C" entry points (abi.cu, noalloc.cu).  With no memory checker available in
// every deployment these host-side checks are the guard against a kernel reading the wrong memory.
#pragma once
#include "../../include/aiter_b200.h"
#include "launch.h"

namespace b200 {

inline const char* dtype_name(int d)
{
    static const char* names[] = {"fp8", "fp8_e8m0", "fp16", "bf16", "fp32", "i4x2", "fp4x2",
                                  "u32", "i32", "i16", "i8", "u8", "i64", "u64"};
    return (d >= 0 && d < 14) ? names[d] : "?";
}

inline bool is_byte_dtype(int d)
{
    return d == AITER_DTYPE_fp8 || d == AITER_DTYPE_fp8_e8m0 || d == AITER_DTYPE_fp4x2 || d == AITER_DTYPE_u8 ||
           d == AITER_DTYPE_i8 || d == AITER_DTYPE_i4x2;
}

inline void require_tensor(const aiter_tensor_t* t, const char* fn, const char* name, int ndim)
{
    B200_CHECK(t != nullptr, fn, ": ", name, " is required");
    B200_CHECK(t->ndim == ndim, fn, ": ", name, " must be ", ndim, "-D (got ", t->ndim, "-D)");
    B200_CHECK(t->device_id >= 0, fn, ": ", name, " must live on a GPU");
    B200_CHECK(t->ptr != nullptr || t->numel_ == 0, fn, ": ", name, " has a null data pointer");
}

// every tensor of one call must live on the same GPU
inline void require_same_device(const aiter_tensor_t* a, const aiter_tensor_t* b, const char* fn, const char* name)
{
    B200_CHECK(b == nullptr || b->device_id == a->device_id, fn, ": ", name, " lives on device ", b ? b->device_id : -1,
               ", the first operand on device ", a->device_id);
}

inline void require_rows_contiguous(const aiter_tensor_t* t, const char* fn, const char* name)
{
    B200_CHECK(t->strides[t->ndim - 1] == 1 || t->shape[t->ndim - 1] == 1, fn, ": ", name,
               " must be contiguous along its last dimension");
}

inline void require_dense(const aiter_tensor_t* t, const char* fn, const char* name)
{
    int64_t expect = 1;
    for(int d = t->ndim - 1; d >= 0; --d)
    {
        B200_CHECK(t->shape[d] == 1 || t->strides[d] == expect, fn, ": ", name, " must be contiguous");
        expect *= t->shape[d];
    }
}

inline ScaleOperand scale_operand(const aiter_tensor_t* s, int wire, const char* fn, const char* name)
{
    require_tensor(s, fn, name, 2);
    B200_CHECK(is_byte_dtype(s->dtype_), fn, ": ", name, " must be e8m0 / uint8 (got ", dtype_name(s->dtype_), ")");
    require_dense(s, fn, name);
    ScaleOperand so;
    so.ptr         = s->ptr;
    so.wire        = wire;
    so.padded_rows = s->shape[0];
    so.padded_cols = s->shape[1];
    return so;
}

} // namespace b200
