"""B200 (sm_100a) implementation of VerseNext's speculative-decoding path.

Public surface (names follow the reference):
  SpeculativeDecoder                      verse_nex/speculative.py:55
  VerseNexLM (= CometSparkNexLM), KVCache verse_nex/cometspark.py:294, kv_cache_parallel.py:42
  build_verse_delta_pattern               verse_nex/delta_attention.py:1218 (layer kinds vda / dsa / kda / gmla)
  SpecEngine                              batched draft -> verify -> accept -> commit loop
  TreeSpecEngine                          the same with tree proposals (greedy rule)
  ShardedSpecEngine, Comm, rank_seed      the same with the LM head split by vocabulary columns over NCCL ranks
  VNFileReader, load_vn                   verse_torch/vn_format.py:527 (.vn container)
  get_backend / clear_backend_cache,
  DeviceBackend, B200Backend              verse_torch/device.py:219-389
  Context, DeviceArray                    device memory (plays torch.Tensor's role, tensor.py:394)
  sampling.accept / sample / argmax       acceptance and sampling kernels

Everything computes in libvn_b200.so; importing this package does not need a
GPU, calling it does.
"""

from . import _lib
from .device import Context, DeviceArray, as_device
from .backend import DeviceBackend, B200Backend, get_backend, clear_backend_cache
from .speculative import SpeculativeDecoder, Tensor, no_grad
from .model import VerseNexLM, CometSparkNexLM, KVCache, build_verse_delta_pattern
from .engine import SpecEngine
from .tree_engine import TreeSpecEngine
from .comm import Comm
from .sharded_engine import ShardedSpecEngine, rank_seed
from .vn_file import VNFileReader, load_vn
from . import sampling
from . import quant

__all__ = ["Context", "DeviceArray", "as_device", "DeviceBackend", "B200Backend", "get_backend",
           "clear_backend_cache", "SpeculativeDecoder", "Tensor", "no_grad", "sampling", "quant", "VerseNexLM", "CometSparkNexLM", "KVCache", "build_verse_delta_pattern", "SpecEngine", "TreeSpecEngine",
           "ShardedSpecEngine", "Comm", "rank_seed", "VNFileReader", "load_vn"]
