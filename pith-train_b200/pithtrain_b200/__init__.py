"""B200-native (sm_100a) context-parallel ring attention behind PithTrain's operator API."""

__version__ = "0.1.0"
