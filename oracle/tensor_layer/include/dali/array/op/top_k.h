// resolves the reference's include path; the declarations live in off_path_ops.h
#include "dali/array/op/off_path_ops.h"
