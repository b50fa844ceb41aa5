// Bounds checks of the debug build (compile with -DPB_BOUNDS_CHECK: `PIPPY_BOUNDS_CHECK=1 python -m pippy_b200.csrc.build`).
//
// Kernels that index memory with values read from tensors (token ids, class labels) validate them in this build:
// an index outside its table sets the device error word to ERR_BOUNDS (5) and the access is skipped, so the
// kernel finishes and the context stays usable; ops._lib.check_device_errors() then raises.  Nothing traps and
// nothing asserts on the device.  In the regular build the macros expand to nothing and the kernels carry no check.
// compute-sanitizer's memcheck does this job where it is available; this build is for where it is not.
#pragma once

extern "C" int* pb_debug_err_ptr();  // common.cu: the error word the host registered (null until it did)

#ifdef PB_BOUNDS_CHECK
#define PB_DBG_PARAMS , int* dbg_err, long long dbg_limit
#define PB_DBG_ARGS(limit) , pb_debug_err_ptr(), (long long)(limit)
// true when idx is a valid row of a table of dbg_limit rows; otherwise records the violation
#define PB_DBG_IN_RANGE(idx) \
  (((idx) >= 0 && (long long)(idx) < dbg_limit) ? true : ((dbg_err ? (void)atomicExch(dbg_err, 5) : (void)0), false))
#else
#define PB_DBG_PARAMS
#define PB_DBG_ARGS(limit)
#define PB_DBG_IN_RANGE(idx) true
#endif
