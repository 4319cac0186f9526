// Observation<Args...>: a list of callbacks that notify() calls in order; ObserverGuard registers one for its own
// lifetime.  Same names and meaning as dali/utils/observer.h:7-55 of the reference (what its Scope and its
// debug::array_as_contiguous hooks are built on), written as one small header.
#ifndef DALI_UTILS_OBSERVER_H
#define DALI_UTILS_OBSERVER_H

#include <functional>
#include <list>
#include <utility>

template <typename... Args> struct ObserverGuard;

template <typename... Args>
struct Observation {
    typedef ObserverGuard<Args...> guard_t;
    typedef std::function<void(Args...)> callback_t;
    typedef typename std::list<callback_t>::iterator callback_handle_t;

    callback_handle_t observe(callback_t callback) {
        callbacks_.push_back(std::move(callback));
        return std::prev(callbacks_.end());
    }
    void lose_interest(callback_handle_t handle) { callbacks_.erase(handle); }
    // calls every observer; returns how many there were
    int notify(Args... args) {
        int n = 0;
        for (auto it = callbacks_.begin(); it != callbacks_.end();) {
            auto next = std::next(it);          // an observer may unregister itself while it is being called
            (*it)(args...);
            ++n;
            it = next;
        }
        return n;
    }
    int num_observers() const { return (int)callbacks_.size(); }

  private:
    std::list<callback_t> callbacks_;
};

template <typename... Args>
struct ObserverGuard {
    Observation<Args...>* dc;
    typename Observation<Args...>::callback_handle_t dc_handle;

    ObserverGuard(typename Observation<Args...>::callback_t callback, Observation<Args...>* dc_)
        : dc(dc_), dc_handle(dc_->observe(std::move(callback))), owns_handle_(true) {}
    ~ObserverGuard() { if (owns_handle_) dc->lose_interest(dc_handle); }
    ObserverGuard(ObserverGuard&& other) : dc(other.dc), dc_handle(other.dc_handle), owns_handle_(other.owns_handle_) {
        other.owns_handle_ = false;
    }
    ObserverGuard(const ObserverGuard&) = delete;
    ObserverGuard& operator=(const ObserverGuard&) = delete;

  private:
    bool owns_handle_;
};

template <typename... Args>
ObserverGuard<Args...> make_observer_guard(typename Observation<Args...>::callback_t callback, Observation<Args...>* dc) {
    return ObserverGuard<Args...>(std::move(callback), dc);
}

#endif
