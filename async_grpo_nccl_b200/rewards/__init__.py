from .registry import REWARD_ADAPTERS, RewardType, get_reward_adapter, register_reward, resolve_adapter  # noqa: F401
from .verifier_pool import VerifierPool, compute_cosine_reward, get_or_create_verifier_pool  # noqa: F401
