"""Runtime utilities around the model and the transport (each module imports on its own):

``prefetch``     pinned host -> device prefetch one step ahead, deferred scalar reads
``graphs``       CUDA-graph capture of a launch-bound forward
``trace``        NVTX ranges and per-phase device spans (``TERRACE_TRACE``)
``health``       heartbeat failure detection over a ``torch.distributed`` store
``drift_probe``  value-level drift instrument (``TERRACE_DRIFT_PROBE``)
"""
