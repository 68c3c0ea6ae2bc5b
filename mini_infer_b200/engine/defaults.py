"""Engine-wide defaults that are not properties of a model."""

# Tokens per cache page.  The reference fixes 16 (src/core/allocator.h:78).
DEFAULT_PAGE_SIZE = 16
