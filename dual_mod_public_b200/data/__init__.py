from .packed import PackedLoader, SyntheticStream, memmap_stream, write_corpus

__all__ = ["PackedLoader", "SyntheticStream", "memmap_stream", "write_corpus"]
