// Named-tensor container and the two checkpoint file formats of the reference
// (src/engine/model/checkpoint.rs): v1 text and v2 binary.  Pure host code.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace vb {

struct CheckpointEntry {
    std::string name;
    std::vector<int64_t> shape;
    std::vector<float> data;
};

struct Checkpoint {
    std::vector<CheckpointEntry> entries;

    const CheckpointEntry *find(const std::string &name) const;
    // replaces an entry of the same name (the reference keeps a map)
    void put(const std::string &name, const std::vector<int64_t> &shape, const float *data, size_t count);
};

// v1 text (checkpoint.rs:14-44): "#volta-checkpoint:v1", "#writer:...", then one line per tensor,
// sorted by name: name|d0,d1,...|v0,v1,...   Values are written with nine significant digits, which
// restores every f32 exactly; the reference's fixed nine decimals are read back just the same.
// v2 binary (checkpoint.rs:162-213): magic "VOLTA\2\0\0", then a zlib stream of stored (uncompressed)
// deflate blocks holding entry_count u32, and per entry name_len u16, name, ndim u32, dims u32 each,
// n_elems u32, f32 data, all little endian.
bool checkpoint_save(const Checkpoint &ck, const std::string &path, int format, std::string *err);
// Reads either format (v2 by its magic; v1 with or without its header line, '#' lines skipped,
// an unknown version refused: checkpoint.rs:46-106, 215-266).
bool checkpoint_load(Checkpoint *ck, const std::string &path, std::string *err);
// The same for a file's bytes already in memory.
bool checkpoint_parse(Checkpoint *ck, const std::string &raw, std::string *err);

// A 64-bit counter as three floats holding 22, 22 and 20 bits, each an exact integer in f32.
void split_u64(uint64_t v, float out[3]);
bool join_u64(const float in[3], uint64_t *v);

}  // namespace vb
