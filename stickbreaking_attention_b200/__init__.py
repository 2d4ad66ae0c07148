"""B200-native stick-breaking attention: drop-in for ``from stickbreaking_attention import sb_attn, sb_attn_varlen``."""
from .sb_attn import sb_attn
from .sb_varlen import sb_attn_varlen
from .ops import check_status, get_carry_policy, get_path, launch_count, set_carry_policy, set_path

__all__ = ["sb_attn", "sb_attn_varlen", "check_status", "set_path", "get_path", "launch_count", "set_carry_policy",
           "get_carry_policy"]
