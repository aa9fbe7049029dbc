/*
 * The reference's inference entry point, as exported by the per-model inference library that
 * `volta-b200-codegen --infer` emits.  Signature of the function the reference's LLVM code
 * generator builds (src/engine/ir/codegen/inner.rs:194-198 in the Volta tree; called as in
 * examples/bench_infer.c:16, 33-47): the model's weights are embedded in the library, `input`
 * holds in_n floats (rows x L0, row-major), `output` receives out_n floats (rows x Ln).
 * The reference compiles one fixed shape; here any whole number of rows is accepted and the
 * call is a no-op when the lengths do not fit the model (the reference has no error channel;
 * volta_b200_last_error(NULL) keeps the reason).  Host or device pointers.  Calls are serialised
 * inside the library.
 */
#ifndef VOLTA_INFER_H
#define VOLTA_INFER_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

void volta_infer(float *input, int64_t in_n, float *output, int64_t out_n);

#ifdef __cplusplus
}
#endif
#endif /* VOLTA_INFER_H */
