// Graph rewrites applied before an expression is lowered (reference: dali/array/expression/optimization.h:8-16,
// optimization.cpp:71-99,144-158).  register_optimization adds a (condition, transformation) pair; canonical()
// walks the value bottom-up, replaces every node for which a condition holds by its transformation, and makes the
// value an assignment into a fresh buffer when it is not one already.  The fusion the reference registers here as
// "jit_merge" (dali/array/jit/jit.cpp:1080-1142,1302) needs no registration on this back end: a whole assignment is
// lowered to one kernel by construction.
#ifndef DALI_ARRAY_EXPRESSION_OPTIMIZATION_H
#define DALI_ARRAY_EXPRESSION_OPTIMIZATION_H

#include <functional>
#include <string>
#include <vector>

#include "dali/array/array.h"

// the arguments of the value assigned by an assignment node
const std::vector<Array>& right_args(Array node);

int register_optimization(std::function<bool(const Array&)> condition, std::function<Array(const Array&)> transformation,
                          const std::string& name);

Array canonical(const Array& array);

#endif
