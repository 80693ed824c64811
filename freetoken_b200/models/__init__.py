"""Model assembly (:mod:`model`) and the architectures the registry knows."""
