"""Import path of the reference (nabla/ops/communication/transfer.py); the ops of this package live in
``collectives.py`` and are re-exported here."""
from . import TransferOp, to_device, transfer_to, cpu, gpu, accelerator  # noqa: F401

__all__ = ['TransferOp', 'to_device', 'transfer_to', 'cpu', 'gpu', 'accelerator']
