"""Mask builders of the pair block (the reference's ``oops.mask``): the producer of triangle attention's ``mask``."""

from .pair_mask_from_token_mask import pair_mask_from_token_mask

__all__ = ["pair_mask_from_token_mask"]
