"""bloomery_b200: a Blackwell-native mixture-of-experts inference server.

Layers (bottom up): ``formats`` (GGUF / safetensors / block quantisation), ``ops``
(ctypes faces of the sm_100a kernels and the CPU library), ``models`` (specs, weights,
CPU oracle), ``runtime`` (engine, KV pool, graphs, residency), ``parallel`` (TP / EP over
NVLink), ``serve`` (HTTP API), ``utils`` (levers, records, flags).
"""
__version__ = "0.1.0"
