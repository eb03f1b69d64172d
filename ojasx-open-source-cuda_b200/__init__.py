"""B200-native (sm_100a) implementation of the ternary-E8 quantized-linear path.

Public names mirror the reference's ``ojasx3.lattice`` / ``ojasx2.streaming_e8`` /
``ojasx3.hardware`` entry points for this path.  The package directory name contains hyphens, so
import it with ``importlib.import_module("ojasx-open-source-cuda_b200")``.
"""

from . import _cabi, ops                                                     # noqa: F401
from .lattice import (E8LatticeLinear, E8LatticePacker, E8QuantizationAwareLinear, RootE8LatticePacker, TernaryE8LatticePacker, _E8STEFunction,   # noqa: F401
                      _FusedE8GEMMFunction, _get_ternary_e8_luts, conway_sloane_e8_project, fwht_block32, pack_model_e8)
from .streaming_e8 import (StreamingE8LoadReport, _copy_row_block_into_layer, _pack_row_block,   # noqa: F401
                           _stream_safetensor_weight, _validate_row_layout, load_hf_checkpoint_e8,
                           pack_weight_rowwise)
from .hardware import (dispatch_tilelang_e8_gemm, fused_ternary_e8_gemm_bwd_dx, fused_ternary_e8_gemm_fwd,     # noqa: F401
                       install_into_reference)
from .sharding import ColumnShardedLinear, shard_rows                        # noqa: F401
from . import torch_ops                                                      # noqa: F401

torch_ops.register()       # torch.ops.ojasx_math_native.fused_ternary_e8_gemm_fwd / _bwd_dx (CUDA, fake, autograd)

__all__ = [
    "E8LatticeLinear", "TernaryE8LatticePacker", "E8LatticePacker", "RootE8LatticePacker", "_FusedE8GEMMFunction", "pack_model_e8", "fwht_block32", "conway_sloane_e8_project", "E8QuantizationAwareLinear",
    "pack_weight_rowwise", "load_hf_checkpoint_e8", "StreamingE8LoadReport", "dispatch_tilelang_e8_gemm", "install_into_reference",
    "fused_ternary_e8_gemm_fwd", "fused_ternary_e8_gemm_bwd_dx", "ColumnShardedLinear",
    "shard_rows", "ops",
]
