"""B200-native (sm_100a) attention / KV-cache path of Token Rush: FP8 KV append-on-write,
split-K flash-decoding with a fused combine, the M-row speculative-verify variant with
device-side commit, the DFlash ring / window attention, chunked prefill attention and
sequence-sharded decode over NVLink.  Host code is Python + PyTorch (tensors, streams,
torch.distributed); all GPU work is hand-written CUDA behind the C ABI in include/trb_kv.h.
"""
from . import _lib, config, fused, ops, state       # noqa: F401
from .config import AttnConfig                      # noqa: F401
from .state import State                            # noqa: F401

__all__ = ["fused", "ops", "state", "config", "AttnConfig", "State"]
