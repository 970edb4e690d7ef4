"""Dataset preprocessing: raw text / instruction data -> tokenised, memory-mapped indexed datasets."""
from .indexed_dataset import IndexedDatasetBuilder, MMapIndexedDataset
from .data_handler import AlpacaHandler, GeneralPretrainHandler, SharegptHandler, get_handler

__all__ = ["IndexedDatasetBuilder", "MMapIndexedDataset", "GeneralPretrainHandler", "AlpacaHandler", "SharegptHandler", "get_handler"]
