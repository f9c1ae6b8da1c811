/* see tensorflow/core/framework/op_kernel.h in this directory */
#include "tensorflow/core/framework/op_kernel.h"
