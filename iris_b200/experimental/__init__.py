"""Experimental features (placeholder namespace, as in the reference's iris/experimental)."""
