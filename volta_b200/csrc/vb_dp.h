// Data-parallel gradient exchange: a thin wrapper over NCCL, loaded at run time with
// dlopen so that single-GPU users need no NCCL at all.  The reference has no collective
// of any kind (no NCCL/MPI/Gloo call site in its tree); this is new functionality whose
// parity target is the single-process result on the full batch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace vb {

class DpComm {
public:
    DpComm() = default;
    ~DpComm();
    // 0 on success. `id` is the 128-byte NCCL unique id shared by all ranks.
    int init(const uint8_t id[128], int world, int rank);
    // In-place sum over ranks of `count` floats, enqueued on `stream` (capturable).
    int all_reduce_sum(float *buf, int64_t count, cudaStream_t stream);
    const std::string &error() const { return err_; }
    static int unique_id(uint8_t out[128], std::string *why = nullptr);

private:
    void *comm_ = nullptr;
    std::string err_;
};

}  // namespace vb
