"""Command-line tools shipped with the framework (run as ``python -m mxnet_b200.tools.<name>``):

``im2rec``     make image lists and pack images into RecordIO files (reference: tools/im2rec.py)
``rec2idx``    rebuild the ``.idx`` file of a ``.rec`` file (reference: tools/rec2idx.py)
``parse_log``  tabulate train/validation metrics from a training log (reference: tools/parse_log.py)
``flakiness_checker``  run one test repeatedly with different seeds (reference: tools/flakiness_checker.py)
``diagnose``   report platform, Python, framework, build and GPU information (reference: tools/diagnose.py)

The multi-process launcher is ``mxnet_b200.parallel.launch`` and the all-reduce bandwidth tool
``mxnet_b200.kvstore.bandwidth`` (reference: tools/launch.py, tools/bandwidth/measure.py)."""
