"""B200 (sm_100a) delta-rule linear-attention kernels behind the LinearNexus op signatures.

``from linearnexus_b200 import gated_delta_rule_chunkwise`` is the drop-in for
``linearnexus.modules.linear_attn.gated_delta_rule_chunkwise`` (torch CUDA tensors instead of
jax arrays).  The compute lives in ``libdeltarule_sm100.so`` (C ABI: include/deltarule_sm100.h).
"""

from .backend import KernelBackend, backend_availability, select_kernel_backend
from .ops import (delta_rule_chunkwise, delta_rule_recurrent, delta_rule_recurrent_pallas,
                  delta_rule_step, gated_delta_rule_chunkwise, gated_delta_rule_recurrent,
                  gated_delta_rule_step, kda_chunkwise, kda_recurrent, kda_step)
from .state import DeltaNetState, GatedDeltaNetState, KDAState
from .host_pipeline import HostPipeline, chunkwise_from_host
from .ops import check_device_status
from .varlen import chunk_backward_varlen, chunkwise_varlen, compute_unpadded_indices, pad, unpad
from .recurrences import (dplr_delta_rule_recurrent, dplr_delta_rule_step, rwkv6_chunkwise, rwkv6_recurrent,
                          rwkv6_step, ssd_chunk_scan, ssd_recurrent_step)
from .block_ops import (depthwise_conv1d_causal, gated_deltanet_gates, kda_gate, rmsnorm_gated,
                        short_conv_silu)

__all__ = [
    "delta_rule_recurrent", "delta_rule_chunkwise", "delta_rule_step", "delta_rule_recurrent_pallas",
    "gated_delta_rule_recurrent", "gated_delta_rule_chunkwise", "gated_delta_rule_step",
    "kda_recurrent", "kda_chunkwise", "kda_step",
    "DeltaNetState", "GatedDeltaNetState", "KDAState",
    "KernelBackend", "backend_availability", "select_kernel_backend",
    "HostPipeline", "chunkwise_from_host", "check_device_status",
    "chunkwise_varlen", "chunk_backward_varlen", "compute_unpadded_indices", "unpad", "pad",
    "dplr_delta_rule_recurrent", "dplr_delta_rule_step", "rwkv6_recurrent", "rwkv6_chunkwise", "rwkv6_step",
    "ssd_chunk_scan", "ssd_recurrent_step",
    "depthwise_conv1d_causal", "short_conv_silu", "gated_deltanet_gates", "kda_gate", "rmsnorm_gated",
]
