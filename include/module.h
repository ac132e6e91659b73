/* Compatibility shim: dnn.c callers include "module.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_MODULE_H
#define DNN_B200_SHIM_MODULE_H
#include "dnn_b200.h"
#endif
