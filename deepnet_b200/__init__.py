"""b200mat: an sm_100a backend for the contrastive-divergence hot path of deepnet.

`deepnet_b200.b200mat` is the `cm` module (the cudamat CUDAMatrix API over
libb200mat.so), `deepnet_b200.dbm` the RBM/DBM training step issued call by call,
`deepnet_b200.fused_rbm` the same step on the fused entry points.
"""
