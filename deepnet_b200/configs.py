"""The five benchmark configurations as (model spec, hyper-parameters, data) builders.

Seeds: data 1000 + config, parameters 2000 + config, random stream 3000 + config.
`cases` bounds the number of synthetic training cases generated (the full data sets
are 60000 / 200000 / 100000 / 60000 / 1000000 cases; a few minibatches suffice for
timing and parity, and every minibatch is drawn from the same generator).
"""
from . import synthetic
from .dbm import CD, PCD, LINEAR, LOGISTIC, REPLICATED_SOFTMAX, Hyperparams

NAMES = {
    0: "c0 binary RBM 784x500 CD-1 B=100",
    1: "c1 Gaussian-binary RBM 1024x4096 CD-1 B=256",
    2: "c2 replicated-softmax RBM 10000x512 CD-1 B=100",
    3: "c3 DBM 784-500-1000 PCD mf=10 gibbs=5 B=100",
    4: "c4 binary RBM 8192x8192 CD-10 B=4096/GPU",
}


def build(config, cases=None, dims_scale=1.0):
    """Returns a dict: layers, edges, hyperparams, batchsize, optimizer, data (dims x cases), seed.

    dims_scale < 1 shrinks the layer sizes (kept multiples of 4) for quick parity cases.
    """
    def d(n):
        return max(4, int(round(n * dims_scale / 4.0)) * 4)

    pseed, dseed, rseed = 2000 + config, 1000 + config, 3000 + config
    if config == 0:
        V, H, B = d(784), d(500), 100
        hyp = Hyperparams(base_epsilon=0.1, initial_momentum=0.5, final_momentum=0.9, momentum_change_steps=3000,
                          gibbs_steps=1)
        ehyp = hyp.copy(apply_l2_decay=True, l2_decay=2e-4)
        data, _ = synthetic.binary_data(V, cases or 60000, dseed)
        layers = [dict(name="v", activation=LOGISTIC, numdims=V, is_input=True),
                  dict(name="h", activation=LOGISTIC, numdims=H)]
        edges = [dict(node1="v", node2="h", weight=synthetic.weights(V, H, 0.01, pseed), hyperparams=ehyp)]
        opt = CD
    elif config == 1:
        V, H, B = d(1024), d(4096), 256
        hyp = Hyperparams(base_epsilon=0.001, initial_momentum=0.9, final_momentum=0.9, gibbs_steps=1)
        data = synthetic.gaussian_data(V, cases or 200000, dseed)
        layers = [dict(name="v", activation=LINEAR, numdims=V, is_input=True),
                  dict(name="h", activation=LOGISTIC, numdims=H)]
        edges = [dict(node1="v", node2="h", weight=synthetic.weights(V, H, 0.001, pseed))]
        opt = CD
    elif config == 2:
        V, H, B = d(10000), d(512), 100
        hyp = Hyperparams(base_epsilon=0.01, initial_momentum=0.9, final_momentum=0.9, gibbs_steps=1,
                          sample_input=True)
        data = synthetic.document_counts(V, cases or 100000, dseed, mean_len=max(4, int(100 * dims_scale)))
        layers = [dict(name="v", activation=REPLICATED_SOFTMAX, numdims=V, is_input=True),
                  dict(name="h", activation=LOGISTIC, numdims=H)]
        edges = [dict(node1="v", node2="h", weight=synthetic.weights(V, H, 0.01, pseed))]
        opt = CD
    elif config == 3:
        V, H1, H2, B = d(784), d(500), d(1000), 100
        hyp = Hyperparams(base_epsilon=0.005, initial_momentum=0.5, final_momentum=0.9, momentum_change_steps=3000,
                          mf_steps=10, gibbs_steps=5)
        data, _ = synthetic.binary_data(V, cases or 60000, dseed)
        layers = [dict(name="v", activation=LOGISTIC, numdims=V, is_input=True),
                  dict(name="h1", activation=LOGISTIC, numdims=H1),
                  dict(name="h2", activation=LOGISTIC, numdims=H2)]
        edges = [dict(node1="v", node2="h1", weight=synthetic.weights(V, H1, 0.01, pseed)),
                 dict(node1="h1", node2="h2", weight=synthetic.weights(H1, H2, 0.01, pseed + 100))]
        opt = PCD
    elif config == 4:
        V, H, B = d(8192), d(8192), 4096
        hyp = Hyperparams(base_epsilon=0.05, initial_momentum=0.9, final_momentum=0.9, gibbs_steps=10)
        data, _ = synthetic.binary_data(V, cases or 1000000, dseed)
        layers = [dict(name="v", activation=LOGISTIC, numdims=V, is_input=True),
                  dict(name="h", activation=LOGISTIC, numdims=H)]
        edges = [dict(node1="v", node2="h", weight=synthetic.weights(V, H, 0.01, pseed))]
        opt = CD
    else:
        raise ValueError("config must be 0..4")
    return dict(name=NAMES[config], layers=layers, edges=edges, hyperparams=hyp, batchsize=B, optimizer=opt,
                data=data, seed=rseed)


def flops_per_example(config):
    """Algorithmic GEMM flops per training case: 2*m*n*k per product, split passes not counted."""
    if config == 0:
        return (3 + 2 * 1) * 2 * 784 * 500
    if config == 1:
        return (3 + 2 * 1) * 2 * 1024 * 4096
    if config == 2:
        return (3 + 2 * 1) * 2 * 10000 * 512
    if config == 3:
        vh, hh, mf, k = 784 * 500, 500 * 1000, 10, 5
        return 2 * (mf * (vh + 2 * hh) + 2 * (vh + hh) + vh + k * (2 * vh + 2 * hh))
    if config == 4:
        return (3 + 2 * 10) * 2 * 8192 * 8192
    raise ValueError(config)
