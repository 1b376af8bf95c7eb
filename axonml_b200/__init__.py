"""axonml_b200: a Blackwell-native deep-learning framework with AxonML's API surface."""
__version__ = "0.1.0"
