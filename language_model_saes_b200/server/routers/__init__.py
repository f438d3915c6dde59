"""HTTP routers of the feature / circuit browser."""
