from .api import Tensor, realize_all
from .impl import TensorImpl
