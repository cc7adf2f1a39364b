from .mmap_dataset import (BlendableWeightedSamplingDataset, KaiMMapDataset, MMapDataset, SyntheticTokenDataset,
                           make_labels, parse_data_prefix, write_corpus)

__all__ = ["BlendableWeightedSamplingDataset", "KaiMMapDataset", "MMapDataset", "SyntheticTokenDataset", "make_labels",
           "parse_data_prefix", "write_corpus"]
