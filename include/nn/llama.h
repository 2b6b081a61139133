/* Forwarding header for callers that include "nn/llama.h" (include/nn/llama.h in the C-ML tree,
 * e.g. examples/llama_inference.c:2): the LLaMA entry points are declared in cml_quant_api.h. */
#ifndef CML_B200_FORWARD_NN_LLAMA_H
#define CML_B200_FORWARD_NN_LLAMA_H
#include "../cml_quant_api.h"
#endif
