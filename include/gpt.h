/* Compatibility shim: dnn.c callers include "gpt.h"; the whole API lives in dnn_b200.h. */
#ifndef DNN_B200_SHIM_GPT_H
#define DNN_B200_SHIM_GPT_H
#include "dnn_b200.h"
#endif
