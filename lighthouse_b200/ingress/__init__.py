"""Ways into the backend other than MLIR payload text (the reference's ``lighthouse.ingress``)."""
