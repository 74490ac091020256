/* TEST INFRASTRUCTURE ONLY -- never linked into the product library.
 *
 * The reference's network and NNInfo objects reference a few shmea persistence symbols
 * (SaveFolder / SaveTable, used by NNInfo::load/save, Structure/nninfo.cpp:787-798).  The oracle
 * harness never loads or saves a skeleton, so these are never reached; they exist only so that the
 * unmodified reference objects link.  (The GUI messaging symbols -- ServiceData, GNet::GServer::send,
 * used by the callbacks in Networks/network.cpp:258-357 -- are implemented by the shim: it records the
 * messages so that the harness can hand them out.)  Each stub is named by
 * the Itanium-ABI mangled symbol and aborts loudly if it is ever called.
 */
#include <stdio.h>
#include <stdlib.h>

#define TRAP(sym)                                                        \
	void sym(void)                                                       \
	{                                                                    \
		fprintf(stderr, "oracle shim: unreachable symbol %s called\n", #sym); \
		abort();                                                         \
	}

TRAP(_ZN5shmea10SaveFolder7newItemERKNS_7GStringERKNS_6GTableE)
TRAP(_ZN5shmea10SaveFolder8loadItemERKNS_7GStringE)
TRAP(_ZN5shmea10SaveFolderC1ERKNS_7GStringE)
TRAP(_ZNK5shmea9SaveTable8getTableEv)
