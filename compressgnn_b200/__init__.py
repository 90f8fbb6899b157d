"""compressgnn_b200: B200 (sm_100a) kernels for CompressGNN's data-parallel hot path --
compressed propagation SpMM, LSH cluster, fused reconstruct -- behind the reference's operator
and layer API.

``runtime``   the eight functions of the reference's ``compressgnn_runtime`` extension
``layer``     Compressgnn_SPMM / KPropagate / Compressgnn_Cluster / Compressgnn_Reconstruct
``loader``    CompressGraph / CompressgnnData (CSR and edge-list forms) and the graph preparation
              (grammar compression on the device or on the host, same arrays)
``offline``   numpy front end of the host library (compressor, filters, partitions)
``sample``    neighbour sampling on the compressed graph (the reference's ``compressgnn_sample``)
``dist``      column sharding over several GPUs (ShardedGCN, place_model)
``model``     GNNLayer / GCN, the caller used by the end-to-end configurations

Importing the package does not load CUDA; the first native call does, and fails loudly when
``libcgnn_b200.so`` has not been built (``python -m compressgnn_b200.build``).
"""
__version__ = "0.1.0"
