"""LoRA / QLoRA adapters, NF4 quantisation, fine-tuning checkpoints; ``adamw_init`` / ``adamw_update``
are re-exported here because fine-tuning loops import them from this module
(reference: nabla/nn/finetune/__init__.py)."""
from ..optim import adamw_init, adamw_update
from .checkpoint import load_finetune_checkpoint, save_finetune_checkpoint
from .lora import (init_lora_adapter, lora_delta, lora_linear, merge_lora_weight, tree_lora_delta,
                   unmerge_lora_weight)
from .qlora import NF4_CODEBOOK, dequantize_nf4, qlora_linear, quantize_nf4
