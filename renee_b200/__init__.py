"""renee_b200 — a Blackwell-native extreme-classification (XC) trainer.

The package trains a text encoder (data parallel) together with a label-sharded
linear classifier over up to 100M+ labels (model parallel), with the loss-skipping
BCE gradient, split SGD/Adam optimizers, split loss scaling and split gradient
accumulation of microsoft/renee (main.py, dl_base.py), re-designed for NVIDIA B200:

* ``renee_b200.ops``       hand-written sm_100a CUDA kernels (tcgen05/TMEM GEMMs fed by TMA
                           for the classifier step, fused encoder kernels, fused AdamW,
                           fused top-K) and their plain PyTorch oracles.
* ``renee_b200.models``    DistilBERT-style encoder (HF-compatible state_dict keys) and the
                           label-sharded classifier state.
* ``renee_b200.parallel``  process bootstrap, symmetric peer memory, fused collectives,
                           heartbeat watchdog, CPU fake peer-memory backend.
* ``renee_b200.data``      synthetic workloads, XC-repository file formats, collation.
* ``renee_b200.optim``     cosine-warmup schedule, loss-scale state machine, optimizers.
* ``renee_b200.utils``     metrics (P/nDCG/PSP/PSnDCG@k), sharding rule, timing, logging.
"""

__version__ = "0.1.0"
