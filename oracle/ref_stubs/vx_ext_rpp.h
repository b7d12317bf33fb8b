/* Stand-in for the vx_rpp extension header: the reference files compiled for the oracle include it but call
 * nothing of it on the paths that are used. Test infrastructure only. */
