from .balance import lpt_balance, plan_frame_exchange
from .frame_parallel import balanced_vit_forward

__all__ = ["lpt_balance", "plan_frame_exchange", "balanced_vit_forward"]
