"""ferrum_b200 — a Blackwell (B200, sm_100a) native deep-learning framework with FERRUM's API surface."""
__version__ = "0.1.0"
