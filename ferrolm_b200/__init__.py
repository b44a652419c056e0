"""ferrolm_b200: B200 (sm_100a) nearest-neighbour search behind ferrolm's `src/vector` API.

The package is a thin host-side mirror of the reference's Rust interface over the C ABI of
`include/ferrovec.h`; all search code is hand-written CUDA in `csrc/`.
"""
from .vector import (NEIGHBOR, Context, FerrovecError, FlatIndex, Hnsw, HnswParams, IvfPq, IvfPqParams, Metric,
                     datagen, datagen_dev, kmeans_assign, kmeans_train, merge_topk_static, neighbors_from_tensor, normalize, padded,
                     recall)

__all__ = ["NEIGHBOR", "Context", "FerrovecError", "FlatIndex", "Hnsw", "HnswParams", "IvfPq", "IvfPqParams", "Metric",
           "datagen", "datagen_dev", "kmeans_assign", "kmeans_train", "merge_topk_static", "neighbors_from_tensor", "normalize", "padded", "recall"]
