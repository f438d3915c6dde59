"""HTTP server for browsing features and circuits. ``language_model_saes_b200.server.app:app`` is the ASGI app; it
reads its database settings from the environment when imported, so this package does not import it eagerly."""
