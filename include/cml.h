/* Forwarding header: callers of C-ML's quantized-LLM path include "cml.h" (include/cml.h in the
 * C-ML tree, e.g. examples/llama_inference.c:1); everything this library offers under those names
 * is declared in cml_quant_api.h. */
#ifndef CML_B200_FORWARD_CML_H
#define CML_B200_FORWARD_CML_H
#include "cml_quant_api.h"
#endif
