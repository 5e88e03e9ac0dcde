from keys_values_b200.optimize.module_wrapper import AccessWeightsGradients
from keys_values_b200.optimize.model_factory import ModelFromFlatVectorsFactory, names_and_modules_for_shard, clone_model_shard_via_flat_vectors
from keys_values_b200.parallel.dp import GradientReducer as CPUOffloadAccumulateGradients

__all__ = ["AccessWeightsGradients", "ModelFromFlatVectorsFactory", "names_and_modules_for_shard", "clone_model_shard_via_flat_vectors",
           "CPUOffloadAccumulateGradients"]
