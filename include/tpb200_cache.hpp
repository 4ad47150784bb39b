// Budgeted weight cache: device copies of host weights keyed by host address, at most `budget`
// bytes; least-recently-used entries that are not pinned are dropped to make room.  The policy of
// the reference's cachedWeight + --vram-budget (src/gpu/cuda/backend.zig:1376-1445; eviction
// :892-970), without its streaming side (that is tpb_stream_*).  Header-only and free of CUDA:
// the owner supplies `upload` (host bytes -> device object) and `release`.
#ifndef TPB200_CACHE_HPP
#define TPB200_CACHE_HPP

#include <cstddef>
#include <functional>
#include <list>
#include <stdexcept>
#include <string>
#include <unordered_map>

namespace tpb {

// The reference's DeviceOutOfMemory for this path: a weight larger than the budget, or pinned
// weights leaving no room for it.
struct CacheFull : std::runtime_error {
    explicit CacheFull(const std::string &what) : std::runtime_error("DeviceOutOfMemory: " + what) {}
};

template <typename Dev>
class WeightCache {
  public:
    using Upload = std::function<Dev(const void *, size_t)>;
    using Release = std::function<void(Dev &)>;

    // budget 0 = no limit
    WeightCache(Upload upload, Release release, size_t budget = 0)
        : upload_(std::move(upload)), release_(std::move(release)), budget_(budget) {}
    ~WeightCache() { dropAll(); }
    WeightCache(const WeightCache &) = delete;
    WeightCache &operator=(const WeightCache &) = delete;

    void setBudget(size_t budget) { budget_ = budget; }
    size_t budget() const { return budget_; }
    size_t bytes() const { return bytes_; }
    size_t hits = 0, misses = 0, evictions = 0;

    // The device object of `host`; uploaded on a miss (a different size under the same address
    // counts as a miss and replaces the entry).  pin = keep it out of eviction until unpin().
    // As in the reference a weight is identified by address and size only: the caller keeps the
    // host memory alive and unchanged while it is cached.
    Dev &get(const void *host, size_t nbytes, bool pin = false) {
        auto it = map_.find(host);
        if (it != map_.end() && it->second.bytes == nbytes) {
            order_.splice(order_.end(), order_, it->second.pos);   // most recent last
            hits++;
        } else {
            if (it != map_.end()) drop(it);
            misses++;
            makeRoom(nbytes);
            Entry e;
            e.dev = upload_(host, nbytes);
            e.bytes = nbytes;
            e.pos = order_.insert(order_.end(), host);
            it = map_.emplace(host, std::move(e)).first;
            bytes_ += nbytes;
        }
        if (pin) it->second.pins++;
        return it->second.dev;
    }
    void unpin(const void *host) {
        auto it = map_.find(host);
        if (it != map_.end() && it->second.pins > 0) it->second.pins--;
    }
    void dropAll() {
        for (auto &kv : map_) release_(kv.second.dev);
        map_.clear();
        order_.clear();
        bytes_ = 0;
    }

  private:
    struct Entry {
        Dev dev{};
        size_t bytes = 0;
        int pins = 0;
        std::list<const void *>::iterator pos;
    };
    using Map = std::unordered_map<const void *, Entry>;

    void drop(typename Map::iterator it) {
        release_(it->second.dev);
        bytes_ -= it->second.bytes;
        order_.erase(it->second.pos);
        map_.erase(it);
    }
    void makeRoom(size_t need) {
        if (budget_ == 0) return;
        if (need > budget_)
            throw CacheFull("weight of " + std::to_string(need) + " bytes exceeds the budget of " + std::to_string(budget_));
        for (auto o = order_.begin(); o != order_.end() && bytes_ + need > budget_;) {
            auto it = map_.find(*o);
            ++o;                                    // drop() erases the node o pointed at
            if (it->second.pins > 0) continue;
            drop(it);
            evictions++;
        }
        if (bytes_ + need > budget_) throw CacheFull("pinned weights leave no room under the budget");
    }

    Upload upload_;
    Release release_;
    size_t budget_ = 0, bytes_ = 0;
    std::list<const void *> order_;                 // least recently used first
    Map map_;
};

}  // namespace tpb

#endif  // TPB200_CACHE_HPP
