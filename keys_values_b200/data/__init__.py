from keys_values_b200.data.base import DataModule, SFTDataset, common_collate_fn, pad_dataset, get_sft_collate_fn
from keys_values_b200.data.dataloader import MyDataLoader
from keys_values_b200.data.iterators import SimilarSequenceLengthIterator, SimilarSequenceLengthSampler
from keys_values_b200.data.module import SequenceLengthFilteredDataModule, SyntheticLongContext
from keys_values_b200.data.helmet import Helmet
from keys_values_b200.data.longbench_v2 import LongBenchV2

__all__ = ["DataModule", "SFTDataset", "common_collate_fn", "pad_dataset", "get_sft_collate_fn", "MyDataLoader",
           "SimilarSequenceLengthIterator", "SimilarSequenceLengthSampler", "SequenceLengthFilteredDataModule",
           "SyntheticLongContext", "Helmet", "LongBenchV2"]
