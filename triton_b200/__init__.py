"""triton_b200: B200-native (sm_100a) tiled matmul and flash attention behind the
call signatures of the reference's op wrappers."""
from .ops import (GroupedMatmul, HostMatmul, attention, attention_backward, attention_forward,  # noqa: F401
                  attention_old, attention_old_forward, group_gemm_fn, matmul, matmul_chain, quantize_e4m3)
from . import custom_ops  # noqa: F401,E402  registers torch.ops.triton_b200.*
