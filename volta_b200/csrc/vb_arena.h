// Static memory plan for one training handle: every buffer of the step lives at a fixed
// offset inside ONE device allocation.
//
// Mirrors the idea of Volta's memory planner (src/engine/ir/memory_planner.rs:47-144:
// liveness interval per value over the fixed schedule, greedy first-fit offsets, aligned)
// and its reuse rule (src/engine/ir/allocation.rs:78-122: only temporaries and gradients of
// activations share storage; parameters and optimizer state never do).  Alignment is 1 KiB
// instead of 16 B so that every buffer can be the base of a TMA tensor map and of
// 128-byte-swizzled tiles.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

namespace vb {

struct PlanBuffer {
    std::string name;
    int64_t bytes = 0;
    int first_use = 0;     // schedule position of the producing launch
    int last_use = 0;      // schedule position of the last consuming launch
    bool persistent = false;
    int64_t offset = -1;   // filled by plan()
};

class ArenaPlan {
public:
    static constexpr int64_t kAlign = 1024;
    // Returns the index of the new buffer.
    int add(const std::string &name, int64_t bytes, int first_use, int last_use, bool persistent) {
        PlanBuffer b;
        b.name = name;
        b.bytes = round_up(bytes > 0 ? bytes : 1);
        b.first_use = first_use;
        b.last_use = last_use;
        b.persistent = persistent;
        bufs_.push_back(b);
        return (int)bufs_.size() - 1;
    }
    // Assign offsets: persistent buffers first, back to back; then temporaries in order of
    // first use (larger first on ties), each at the lowest offset where it overlaps no
    // already-placed buffer that is live at the same time.
    void plan();
    // True when no two buffers whose lifetimes intersect share a byte (the aliasing check
    // of allocation.rs:147-208), and everything lies inside [0, total).
    bool verify(std::string *why = nullptr) const;
    int64_t total() const { return total_; }
    int64_t offset(int idx) const { return bufs_[idx].offset; }
    int64_t sum_unshared() const;  // bytes if nothing were reused (for reporting)
    const std::vector<PlanBuffer> &buffers() const { return bufs_; }
    static int64_t round_up(int64_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

private:
    std::vector<PlanBuffer> bufs_;
    int64_t total_ = 0;
};

}  // namespace vb
