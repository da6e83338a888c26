from .rdataset import DatasetWorker, RDataset

__all__ = ["DatasetWorker", "RDataset"]
