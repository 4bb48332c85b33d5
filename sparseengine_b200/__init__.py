"""sparseengine_b200: a small, whole inference engine for one GPU (B200, sm_100a)."""
__version__ = "0.1.0"
