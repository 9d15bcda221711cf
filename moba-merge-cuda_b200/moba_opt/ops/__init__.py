"""Standalone operators behind the reference's `moba_opt.ops` names."""
