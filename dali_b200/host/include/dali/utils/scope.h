// Trace scopes (reference: dali/utils/scope.h:11-57, scope.cpp:22-45).  DALI_SCOPE(name) opens a named scope for the
// rest of the enclosing block, but only while somebody observes; a ScopeObserver keeps the stack of open scope names
// and is told when one is entered or left.  Every computation the front end runs opens a scope named after the
// expression it evaluates (dali/array/expression/computation.cpp:14-21), which is how the reference's tests count
// computations to show that an expression stayed lazy (dali/array/tests/dot_tests.cpp:17-35).  Not thread safe, as in
// the reference (scope.h:35).
#ifndef DALI_UTILS_SCOPE_H
#define DALI_UTILS_SCOPE_H

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "dali/utils/observer.h"

#define DALI_SCOPE(str)                                                              \
    std::unique_ptr<Scope> dali_scope_guard_;                                        \
    if (Scope::has_observers()) {                                                    \
        dali_scope_guard_ = std::unique_ptr<Scope>(new Scope(std::make_shared<std::string>(str))); \
    }

struct Scope {
    typedef std::shared_ptr<std::string> name_t;
    static Observation<name_t> obs_enter;
    static Observation<name_t> obs_exit;
    static bool has_observers();

    bool active;
    name_t name;
    Scope();
    explicit Scope(name_t name_);
    ~Scope();
    Scope(const Scope&) = delete;
    Scope& operator=(const Scope&) = delete;
};

struct ScopeObserver {
    struct State { std::vector<Scope::name_t> trace; };
    typedef std::function<void(const State&)> callback_t;
    // either callback may be empty (the reference's tests pass NULL for on_enter)
    ScopeObserver(callback_t on_enter_, callback_t on_exit_);

  private:
    const callback_t on_enter_, on_exit_;
    State state_;
    decltype(Scope::obs_enter)::guard_t enter_guard_;
    decltype(Scope::obs_exit)::guard_t exit_guard_;
};

#endif
