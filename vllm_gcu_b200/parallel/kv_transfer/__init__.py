"""KV-cache transfer: LMCache offload ops and the point-to-point connector for
disaggregated prefill / decode (vllm_gcu/distributed/kv_transfer/, lmcache/csrc/)."""
from . import lmcache_ops  # noqa: F401
from .p2p_connector import P2PKVConnector, TensorMemoryPool  # noqa: F401
