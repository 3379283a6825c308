from . import presets
from .cache import Cached
from .dataset import DataPartition, Dataset, Files, Loader, Memory, TokenFiles, collate
from .mixing import Mixture, PhasedStream, RampedStream
from .packing import Packer, pack_whole
from .sources import Hub, JsonLines, Parquet
from .tokenizer import ByteTokenizer
from . import analysis, holdout, images, shards, video
from .forked_rows import ForkedRows, Forks
from .holdout import Holdout
from .images import Augment, ImageFolder
from .shards import TarShards, write_shards
from .video import Clips

__all__ = ["Dataset", "Memory", "Files", "TokenFiles", "Loader", "DataPartition", "ByteTokenizer", "presets", "collate", "Cached",
           "Packer", "pack_whole", "Hub", "JsonLines", "Parquet", "Mixture", "PhasedStream", "RampedStream", "Holdout", "Augment", "ImageFolder", "TarShards", "write_shards", "Clips",
           "analysis", "holdout", "images", "shards", "video", "ForkedRows", "Forks"]
