from .csr import edge_index_to_csr

__all__ = ["edge_index_to_csr"]
