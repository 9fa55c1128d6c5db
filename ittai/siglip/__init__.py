"""``ittai.siglip`` (a namespace package in the reference): see ``ittai.siglip.kernel``."""
