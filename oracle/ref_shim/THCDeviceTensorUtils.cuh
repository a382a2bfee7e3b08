/* Stand-in for cutorch's THCDeviceTensorUtils.cuh (tensor -> device view helpers live in the host wrappers, unused). */
