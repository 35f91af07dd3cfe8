"""Memory probes built on a Jacobian lens: what the fast-weight memory holds and how it is read."""
