#include "vb_arena.h"

#include <algorithm>

namespace vb {

static bool lives_overlap(const PlanBuffer &a, const PlanBuffer &b) {
    if (a.persistent || b.persistent) return true;
    return a.first_use <= b.last_use && b.first_use <= a.last_use;
}

void ArenaPlan::plan() {
    int64_t top = 0;
    for (auto &b : bufs_)
        if (b.persistent) {
            b.offset = top;
            top += b.bytes;
        }
    const int64_t temp_base = top;
    std::vector<int> order;
    for (int i = 0; i < (int)bufs_.size(); ++i)
        if (!bufs_[i].persistent) order.push_back(i);
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) {
        if (bufs_[x].first_use != bufs_[y].first_use) return bufs_[x].first_use < bufs_[y].first_use;
        return bufs_[x].bytes > bufs_[y].bytes;
    });
    std::vector<int> placed;
    for (int idx : order) {
        PlanBuffer &b = bufs_[idx];
        // candidate offsets: the base and the end of every conflicting placed buffer
        std::vector<int64_t> cands{temp_base};
        for (int p : placed)
            if (lives_overlap(b, bufs_[p])) cands.push_back(bufs_[p].offset + bufs_[p].bytes);
        std::sort(cands.begin(), cands.end());
        for (int64_t c : cands) {
            bool ok = true;
            for (int p : placed) {
                const PlanBuffer &q = bufs_[p];
                if (!lives_overlap(b, q)) continue;
                if (c < q.offset + q.bytes && q.offset < c + b.bytes) {
                    ok = false;
                    break;
                }
            }
            if (ok) {
                b.offset = c;
                break;
            }
        }
        placed.push_back(idx);
        top = std::max(top, b.offset + b.bytes);
    }
    total_ = top;
}

bool ArenaPlan::verify(std::string *why) const {
    for (size_t i = 0; i < bufs_.size(); ++i) {
        const PlanBuffer &a = bufs_[i];
        if (a.offset < 0 || a.offset % kAlign || a.offset + a.bytes > total_) {
            if (why) *why = "buffer '" + a.name + "' lies outside the arena or is misaligned";
            return false;
        }
        for (size_t j = i + 1; j < bufs_.size(); ++j) {
            const PlanBuffer &b = bufs_[j];
            if (!lives_overlap(a, b)) continue;
            if (a.offset < b.offset + b.bytes && b.offset < a.offset + a.bytes) {
                if (why) *why = "buffers '" + a.name + "' and '" + b.name + "' are live together and overlap";
                return false;
            }
        }
    }
    return true;
}

int64_t ArenaPlan::sum_unshared() const {
    int64_t s = 0;
    for (auto &b : bufs_) s += b.bytes;
    return s;
}

}  // namespace vb
