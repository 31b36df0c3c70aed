"""B200-native (sm_100a) LLM inference engine.

PyTorch is the framework layer (model graphs, scheduler, cache manager, sampler, HTTP
surface); the hot ops are hand-written CUDA kernels in ``ops/csrc`` (tcgen05 / TMEM GEMMs fed
by TMA, paged attention, recurrent-state updates, sampling) and the multi-GPU paths fuse
compute with their collectives over NVLink peer memory (``parallel/``).
"""
__version__ = "0.1.0"
