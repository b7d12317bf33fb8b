/* Stand-in for a protobuf-generated header that the reference's metadata readers include; the random-bbox-crop
 * reader compiled for the oracle uses none of its types. Test infrastructure only. */
