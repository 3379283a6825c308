from . import presets
from .dataset import DataPartition, Dataset, Files, Loader, Memory, TokenFiles, collate
from .tokenizer import ByteTokenizer

__all__ = ["Dataset", "Memory", "Files", "TokenFiles", "Loader", "DataPartition", "ByteTokenizer", "presets", "collate"]
