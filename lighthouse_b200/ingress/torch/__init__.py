"""``torch.compile`` entry: the reference's ``lighthouse.ingress.torch`` for this backend."""

from .compile import BufferMetadata, CudaBackend, JITFunction, UnsupportedGraph, gpu_backend, import_fx_graph

__all__ = ["BufferMetadata", "CudaBackend", "JITFunction", "UnsupportedGraph", "gpu_backend", "import_fx_graph"]
