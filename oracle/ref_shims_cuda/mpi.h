/* Stand-in for <mpi.h>: apache/singa's communicator includes it
 * (include/singa/io/communicator.h:26) and calls six MPI routines from the
 * constructor that bootstraps through MPI (src/io/communicator.cc:79-98, 191).
 * No MPI is installed where the comparator is built, and the checker only
 * uses the constructor that receives an NCCL id, so the routines below exist
 * to satisfy the compiler and fail when called.  TEST INFRASTRUCTURE ONLY. */
#ifndef SGB_REF_MPI_H_
#define SGB_REF_MPI_H_
typedef int MPI_Comm;
typedef int MPI_Datatype;
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_COMM_WORLD 0
#define MPI_BYTE 1
#define MPI_DATATYPE_NULL 0
#define MPI_IN_PLACE ((void *)1)
static inline int MPI_Init(int *argc, char ***argv) { (void)argc; (void)argv; return MPI_ERR_OTHER; }
static inline int MPI_Finalize(void) { return MPI_ERR_OTHER; }
static inline int MPI_Comm_rank(MPI_Comm c, int *r) { (void)c; *r = 0; return MPI_ERR_OTHER; }
static inline int MPI_Comm_size(MPI_Comm c, int *s) { (void)c; *s = 1; return MPI_ERR_OTHER; }
static inline int MPI_Allgather(const void *sb, int sc, MPI_Datatype st, void *rb, int rc, MPI_Datatype rt,
                                MPI_Comm c) {
  (void)sb; (void)sc; (void)st; (void)rb; (void)rc; (void)rt; (void)c;
  return MPI_ERR_OTHER;
}
static inline int MPI_Bcast(void *b, int n, MPI_Datatype t, int root, MPI_Comm c) {
  (void)b; (void)n; (void)t; (void)root; (void)c;
  return MPI_ERR_OTHER;
}
#endif
