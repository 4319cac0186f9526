// forwards to the op:: umbrella (reference: dali/array/op/outer.h)
#include "dali/array/op.h"
