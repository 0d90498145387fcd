"""nestor_b200: a Blackwell-native training framework for the Nestor nested sparse transformer.

The package mirrors the capability surface of Ma-Lab-Berkeley/Nestor (``nestor_cli``,
``@register_experiment`` cells, ``DCLM_*`` run knobs, the checkpoint key layout) on
top of a different runtime: parameters live in flat per-dtype arenas, the hot ops
are sm_100a CUDA kernels (``nestor_b200/csrc``), and the data-parallel paths move
gradients and parameter updates through peer memory from inside kernels.
"""

__version__ = "0.1.0"
