"""B200-native fused FP8 block-scale DeepSeek-V3 MoE layer (sm_100a only).

Public surface: :func:`run_moe` (the reference's entry point, same argument order),
:func:`run_moe_host`, :func:`route`, :class:`MoeContext`, and the seeded workload
generator in :mod:`workloads`.
"""
from .moe import (ABI, EpDesc, MoeContext, MoeError, get_context, library_path, load_library, release_contexts, route,
                  run_moe, run_moe_ep, run_moe_ep_replicated, ep_prepare, run_moe_host, ep_region_bytes, PackedWeights, prepack_weights,
                  run_moe_prepacked)
from .dsa import run_dsa_topk_indexer, dsa_check
from .parallel import ExpertParallelMoe, expert_slice
from .workloads import MoeInputs, algorithmic_work, make_inputs

__all__ = ["ABI", "ExpertParallelMoe", "expert_slice", "MoeContext", "MoeError", "MoeInputs", "algorithmic_work", "get_context", "library_path",
           "load_library", "make_inputs", "release_contexts", "route", "run_moe", "run_moe_ep", "run_moe_ep_replicated", "ep_prepare", "run_moe_host",
           "EpDesc", "ep_region_bytes", "PackedWeights", "prepack_weights", "run_moe_prepacked", "run_dsa_topk_indexer", "dsa_check"]
