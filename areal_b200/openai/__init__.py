from .cache import InteractionCache
from .client import ArealOpenAI
from .types import ChatCompletion, InteractionWithTokenLogpReward

__all__ = ["ArealOpenAI", "InteractionCache", "InteractionWithTokenLogpReward", "ChatCompletion"]
