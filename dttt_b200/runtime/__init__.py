"""The pieces a training run is assembled from: operator signals, command-line to configuration, restart planning,
the evaluation suite.  ``dttt_b200.train`` wires them around ``engine.Engine``."""
