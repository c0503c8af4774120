from .managers import (DAPORewardManager, NaiveRewardManager, ParallelRewardManager,  # noqa: F401
                       EmbodiedRewardManager, REWARD_MANAGERS)
