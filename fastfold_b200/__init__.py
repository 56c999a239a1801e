"""fastfold_b200: a Blackwell-native (sm_100a) Evoformer / AlphaFold training and inference framework.

Sub-packages: ``ops`` (kernels), ``parallel`` (DAP runtime), ``models`` (``nn`` OpenFold-layout reference modules,
``fastnn`` fast modules, ``hub`` full model), ``runtime`` (training engine), ``utils``, ``common``, ``data``.
"""
__version__ = "0.1.0"
