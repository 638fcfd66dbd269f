"""Operation layer: collectives, neighbor ops and one-sided windows."""
