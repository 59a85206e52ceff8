// Tensor-core forms of the masked softmax attention (bfloat16): see masked_attention.cu.
#pragma once
