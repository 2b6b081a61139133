/* C-ML's include/nn/llm_ops.h, served by libcml_b200: KV cache, grouped-query attention, RoPE and the BPE tokenizer are declared in cml_quant_api.h (the mixture-of-experts and flash variants of that header are outside this library). */
#ifndef CML_B200_NN_LLM_OPS_H
#define CML_B200_NN_LLM_OPS_H
#include "../cml_quant_api.h"
#endif
