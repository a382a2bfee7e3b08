/* Stand-in for cutorch's type-instantiation header: the generic host wrappers are not instantiated. */
#undef THC_GENERIC_FILE
