from .checkpoint import load_finetune_checkpoint, save_finetune_checkpoint
from .lora import (init_lora_adapter, lora_delta, lora_linear, merge_lora_weight, tree_lora_delta,
                   unmerge_lora_weight)
from .qlora import NF4_CODEBOOK, dequantize_nf4, qlora_linear, quantize_nf4
