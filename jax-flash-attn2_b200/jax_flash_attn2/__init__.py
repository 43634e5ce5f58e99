"""B200-native FlashAttention-2 behind the jax_flash_attn2 API."""
from .flash_attention import (
    AttentionConfig,
    Backend,
    FlashAttention,
    Platform,
    create_flash_attention,
)
from ._flash_attention import flash_attention as triton_flash_attention
from ._kernel_calls import (
    bwd_attention_kernel_call,
    device_status,
    dropout_bits_buffer,
    fwd_attention_kernel_call,
)

__all__ = (
    "AttentionConfig",
    "Backend",
    "FlashAttention",
    "Platform",
    "create_flash_attention",
    "triton_flash_attention",
    "fwd_attention_kernel_call",
    "bwd_attention_kernel_call",
    "device_status",
    "dropout_bits_buffer",
)
__version__ = "0.1.0"
