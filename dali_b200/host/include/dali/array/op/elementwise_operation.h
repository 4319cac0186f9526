// forwards to the op:: umbrella (reference: dali/array/op/elementwise_operation.h)
#include "dali/array/op.h"
