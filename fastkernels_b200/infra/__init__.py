"""Host-side glue mirrored from the reference's fastkernels/infra (decode path only)."""
