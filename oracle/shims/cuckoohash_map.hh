// Test infrastructure only: stand-in for the un-vendored libcuckoo submodule
// (third_party/libcuckoo is an empty directory in the reference checkout).
// Implements just the calls made by dali/array/memory/memory_bank.cpp:42-79
// (upsert, update_fn, cbegin()/is_end()/operator->) on a mutex-guarded
// std::unordered_map.  It carries no arithmetic of the hot path.
#ifndef DALI_B200_ORACLE_CUCKOO_SHIM_H
#define DALI_B200_ORACLE_CUCKOO_SHIM_H
#include <atomic>
#include <mutex>
#include <unordered_map>
#include <utility>

template <typename K, typename V>
class cuckoohash_map {
    std::unordered_map<K, V> map_;
    mutable std::mutex mu_;
  public:
    explicit cuckoohash_map(size_t reserve = 0) { map_.reserve(reserve < 1024 ? reserve : 1024); }

    template <typename F>
    void upsert(const K& key, F fn, V init) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = map_.find(key);
        if (it == map_.end()) map_.emplace(key, std::move(init));
        else fn(it->second);
    }

    template <typename F>
    bool update_fn(const K& key, F fn) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = map_.find(key);
        if (it == map_.end()) return false;
        fn(it->second);
        return true;
    }

    struct const_iterator {
        typename std::unordered_map<K, V>::const_iterator it, end;
        bool is_end() const { return it == end; }
        const std::pair<const K, V>* operator->() const { return &*it; }
        const_iterator operator++(int) { const_iterator c = *this; ++it; return c; }
    };
    const_iterator cbegin() const { return const_iterator{map_.cbegin(), map_.cend()}; }
};
#endif
