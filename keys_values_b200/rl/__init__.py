from keys_values_b200.rl.logprobs import LogProbsHeadModel, compute_logprobs
from keys_values_b200.rl.grpo import GRPOLossHeadModel, compute_group_advantages, grpo_step, generate_completions

__all__ = ["LogProbsHeadModel", "compute_logprobs", "GRPOLossHeadModel", "compute_group_advantages", "grpo_step", "generate_completions"]
