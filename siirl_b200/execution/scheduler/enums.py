"""Enumerations of the control plane (reference: siirl/execution/scheduler/enums.py:18-63)."""
import enum


class AdvantageEstimator(str, enum.Enum):
    GAE = "gae"
    GRPO = "grpo"
    CPGD = "cpgd"
    GAE_MARFT = "gae_marft"


class WorkflowType(str, enum.Enum):
    DEFAULT = "default"
    DAPO = "dapo"
    EMBODIED = "embodied"


class Role(enum.Enum):
    Actor = 0
    Rollout = 1
    ActorRollout = 2
    Critic = 3
    RefPolicy = 4
    RewardModel = 5
    ActorRolloutRef = 6


class AlgorithmType(str, enum.Enum):
    PPO = "ppo"
    GRPO = "grpo"
    DAPO = "dapo"
    GSPO = "gspo"
    CPGD = "cpgd"
    SRPO = "srpo"
    MARFT = "marft"
