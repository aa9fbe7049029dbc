/*
 * The reference's own training-library symbols, as exported by every per-model library
 * that `volta-b200-codegen` emits.  Signatures are those of the reference's generated
 * code (src/engine/ir/codegen/mlp_train_rust_codegen.rs:641-699 in the Volta tree; C twin
 * src/engine/ir/codegen/mlp_train_codegen.rs:112-124), so a host harness written against
 * a Volta training DLL loads the emitted library unchanged.  The bodies forward to
 * libvolta_b200 (include/volta_b200.h) with the model's topology compiled in.
 */
#ifndef VOLTA_TRAIN_H
#define VOLTA_TRAIN_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct vb200_handle VoltaTrainHandle;

/* mlp_train_rust_codegen.rs:641-667. Returns NULL on failure (as the C path does on a
 * failed allocation, mlp_train_codegen.rs:210-211); volta_b200_last_error(NULL) says why. */
VoltaTrainHandle *volta_train_init(int32_t batch);
/* mlp_train_rust_codegen.rs:670-675 */
void volta_train_set_params(VoltaTrainHandle *h, int32_t li, const float *w, const float *b);
/* mlp_train_rust_codegen.rs:678-684: pointers into a host mirror refreshed by this call */
void volta_train_get_params(VoltaTrainHandle *h, float **wo, float **bo);
/* mlp_train_rust_codegen.rs:686 */
float volta_train_loss(VoltaTrainHandle *h);
/* mlp_train_rust_codegen.rs:699: X [batch x L0], Y [batch x Ln], host or device pointers */
void volta_train_step(VoltaTrainHandle *h, const float *X, const float *Y, float lr);
/* mlp_train_rust_codegen.rs:689-696: NULL is a no-op */
void volta_train_free(VoltaTrainHandle *h);

#ifdef __cplusplus
}
#endif
#endif /* VOLTA_TRAIN_H */
