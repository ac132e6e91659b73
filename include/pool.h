/* Compatibility shim: dnn.c callers include "pool.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_POOL_H
#define DNN_B200_SHIM_POOL_H
#include "dnn_b200.h"
#endif
