// forwards to the op:: umbrella (reference: dali/array/op/gather_from_rows.h)
#include "dali/array/op.h"
