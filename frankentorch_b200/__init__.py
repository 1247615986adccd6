"""frankentorch_b200: a Blackwell-native tensor / autograd training framework.

Public surface: :class:`FrankenTorchSession` (handle-based tensor API on the Deterministic
Autograd Contract tape), ``nn`` / ``optim`` / ``data`` / ``serialize`` mirrors, the GPT model
family and training engine on hand-written sm_100a kernels, and the multi-GPU paths in
``parallel``.
"""
from .runtime.ledger import EvidenceEntry, EvidenceKind, ExecutionMode  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # heavy modules are imported on first use so `import frankentorch_b200` stays cheap
    if name == "FrankenTorchSession":
        from .session import FrankenTorchSession
        return FrankenTorchSession
    if name in ("nn", "optim", "data", "serialize", "conformance", "models", "parallel", "ops", "training"):
        import importlib
        return importlib.import_module(f".{name}", __name__)
    raise AttributeError(name)
