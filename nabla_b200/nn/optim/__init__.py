from .functional import adamw_step, sgd_step, sgd_update
from .optimizer import SGD, AdamW, Optimizer, adamw_init, adamw_update
