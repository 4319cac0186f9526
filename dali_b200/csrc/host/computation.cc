// Scopes, the implementation registry and the optimize -> lower -> run driver behind Array::eval
// (reference: dali/utils/scope.cpp:5-45, dali/array/expression/computation.cpp:13-165,
// dali/array/expression/optimization.cpp:71-158).
#include <map>
#include <unordered_set>

#include "../../../include/dali_b200.h"
#include "dali/array/expression/computation.h"
#include "dali/array/expression/expression.h"
#include "dali/array/expression/optimization.h"
#include "dali/utils/scope.h"

// ------------------------------------------------------------------ scopes
Observation<Scope::name_t> Scope::obs_enter;
Observation<Scope::name_t> Scope::obs_exit;

bool Scope::has_observers() { return obs_enter.num_observers() + obs_exit.num_observers() > 0; }
Scope::Scope() : active(false) {}
Scope::Scope(name_t name_) : active(true), name(name_) { obs_enter.notify(name); }
Scope::~Scope() { if (active) obs_exit.notify(name); }

ScopeObserver::ScopeObserver(callback_t on_enter, callback_t on_exit)
    : on_enter_(on_enter), on_exit_(on_exit),
      enter_guard_([this](Scope::name_t name) {
          state_.trace.push_back(name);
          if (on_enter_) on_enter_(state_);
      }, &Scope::obs_enter),
      exit_guard_([this](Scope::name_t) {
          if (on_exit_) on_exit_(state_);
          if (!state_.trace.empty()) state_.trace.pop_back();
      }, &Scope::obs_exit) {}

// ------------------------------------------------------------------ Computation
Computation::Computation(Array left, OPERATOR_T operator_t, Array right, Array assignment)
    : left_(left), operator_t_(operator_t), right_(right), assignment_(assignment) {}

void Computation::run_and_cleanup() {
    {
        std::string assign_name;
        if (Scope::has_observers()) assign_name = right_.full_expression_name();
        DALI_SCOPE(assign_name);
        run();
    }
    // evaluated once, remembered: the assignment node is replaced by what it wrote to (a buffer, or -- after a
    // scatter -- the lazy gather of the updated source)
    if (left_.is_assignment()) left_.eval(false);
    assignment_.set_expression(left_.expression());
}

void* Computation::left_data(memory::Device device) {
    BufferView* b = as<BufferView>(left_);
    DALI_ASSERT(b, "left_data: the destination is not a buffer");
    return (char*)b->memory_->data(device, memory::AM_MUTABLE) + b->offset_ * size_of_dtype(b->dtype_);
}

const void* Computation::argument_data(memory::Device device, int idx) const {
    const std::vector<Array>& args = right_.expression()->arguments_;
    DALI_ASSERT(idx >= 0 && idx < (int)args.size(), "argument_data: the value has no argument " + std::to_string(idx));
    Array a = args[idx];
    if (!a.is_buffer()) a.eval(false);
    BufferView* b = as<BufferView>(a);
    DALI_ASSERT(b, "argument_data: argument " + std::to_string(idx) + " did not evaluate to a buffer");
    return (const char*)b->memory_->data(device, memory::AM_READONLY) + b->offset_ * size_of_dtype(b->dtype_);
}

namespace {

// What every assignment falls back on: the fused-kernel lowering (one generated kernel per assignment, a tensor-core
// GEMM with the surrounding elementwise tree as its epilogue where the value is built around a product).
struct LoweredComputation : public Computation {
    using Computation::Computation;
    void run() override { lazy::run_assignment(left_, operator_t_, right_); }
};

struct ByName { std::vector<to_computation_t> factories; };
struct ByTest { std::string opname; implementation_test_t test; to_computation_t factory; };
struct Optimization { std::function<bool(const Array&)> condition; std::function<Array(const Array&)> transformation; std::string name; };

std::map<std::string, ByName>& implementations() { static auto* m = new std::map<std::string, ByName>(); return *m; }
std::vector<ByTest>& implementations_by_test() { static auto* v = new std::vector<ByTest>(); return *v; }
std::vector<Optimization>& optimizations() { static auto* v = new std::vector<Optimization>(); return *v; }

// post-order: arguments first, then the node itself (dali/array/expression/optimization.cpp:71-99)
void simplify(const Array& a, std::unordered_set<const Expression*>& seen, int depth) {
    if (a.is_stateless() || depth > 256) return;
    expression_ptr e = a.expression();
    if (e->kind_ == N_BUFFER || e->kind_ == N_SCALAR || e->kind_ == N_IOTA) return;
    if (!seen.insert(e.get()).second) return;
    for (const Array& arg : e->arguments_) simplify(arg, seen, depth + 1);
    for (const Optimization& o : optimizations()) {
        if (!o.condition(a)) continue;
        Array replaced = o.transformation(a);
        if (!replaced.is_stateless() && replaced.expression() != a.expression()) a.set_expression(replaced.expression());
    }
}

}  // namespace

int register_implementation(const char* opname, to_computation_t impl) {
    implementations()[opname].factories.push_back(impl);
    return 0;
}

int register_implementation(const std::string& opname, implementation_test_t test, to_computation_t impl) {
    implementations_by_test().push_back(ByTest{opname, test, impl});
    return 0;
}

int register_optimization(std::function<bool(const Array&)> condition, std::function<Array(const Array&)> transformation,
                          const std::string& name) {
    optimizations().push_back(Optimization{condition, transformation, name});
    return 0;
}

const std::vector<Array>& right_args(Array node) {
    Assignment* a = as<Assignment>(node);
    DALI_ASSERT(a, "right_args: not an assignment");
    return a->arguments_[1].expression()->arguments_;
}

Array canonical(const Array& array) {
    DALI_ASSERT(!array.is_stateless(), "canonical() of a stateless Array");
    if (!optimizations().empty()) {
        std::unordered_set<const Expression*> seen;
        simplify(array, seen, 0);
    }
    expression_ptr e = array.expression();
    if (e->kind_ == N_BUFFER || e->kind_ == N_ASSIGN) return array;
    // wrap the value in an assignment to a fresh buffer (optimization.cpp:29-67 does this for every node that is not
    // assignable; here only the root needs it -- what cannot share the root's kernel is given its own assignment
    // during lowering).  The buffer is the same part of a logical array as the value.
    const memory::Device device = e->kind_ == N_SCALAR ? memory::default_preferred_device : array.preferred_device();
    Array dest(e->shape_, e->dtype_, device);
    dest.expression()->shard_ = e->shard_;
    array.set_expression(std::make_shared<Assignment>(dest, OPERATOR_T_EQL, Array(e)));
    return array;
}

std::vector<std::shared_ptr<Computation>> convert_to_ops(Array root) {
    std::vector<std::shared_ptr<Computation>> steps;
    if (root.is_stateless() || !root.is_assignment()) return steps;
    Assignment* a = static_cast<Assignment*>(root.expression().get());
    Array left = a->arguments_[0], right = a->arguments_[1];
    std::shared_ptr<Computation> step;
    if (!right.is_stateless()) {
        const Expression& node = *right.expression();
        auto it = implementations().find(typeid(node).name());
        if (it != implementations().end())
            for (const to_computation_t& make : it->second.factories) {
                step = make(left, a->operator_t_, right, root);
                if (step) break;
            }
        if (!step)
            for (const ByTest& t : implementations_by_test()) {
                if (!t.test(right)) continue;
                step = t.factory(left, a->operator_t_, right, root);
                if (step) break;
            }
    }
    if (!step) step = std::make_shared<LoweredComputation>(left, a->operator_t_, right, root);
    steps.push_back(step);
    return steps;
}
