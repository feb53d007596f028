"""Entry points: the offline-batch command line."""
