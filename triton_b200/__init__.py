"""triton_b200: B200-native (sm_100a) tiled matmul and flash attention behind the
call signatures of the reference's op wrappers."""
from .ops import GroupedMatmul, HostMatmul, group_gemm_fn, attention, attention_backward, attention_forward, matmul, matmul_chain, quantize_e4m3  # noqa: F401
from . import custom_ops  # noqa: F401,E402  registers torch.ops.triton_b200.*
