from .mmap_dataset import (BlendableWeightedSamplingDataset, KaiMMapDataset, MMapDataset, SyntheticTokenDataset,
                           make_labels, parse_data_prefix, write_corpus)
from .loader import ResumableLoader
from .parquet_dataset import DistributedParquetDataset, ParquetReader, ShuffledParquetReader, expand_sources

__all__ = ["BlendableWeightedSamplingDataset", "KaiMMapDataset", "MMapDataset", "SyntheticTokenDataset", "make_labels",
           "parse_data_prefix", "write_corpus", "DistributedParquetDataset", "ParquetReader", "ShuffledParquetReader",
           "expand_sources", "ResumableLoader"]
