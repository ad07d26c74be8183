/* A single-node MPI subset over shared memory, just large enough to build and run the
 * reference's communication library (fflib2) and its evaluation programs unmodified on a
 * machine that has no MPI installation.
 *
 * Covered: Init / Init_thread (MPI_THREAD_MULTIPLE) / Initialized / Finalize, Comm_rank /
 * Comm_size on MPI_COMM_WORLD, Isend / Irecv with (source, tag) matching in posting order,
 * Test / Testsome / Wait / Waitsome / Cancel / Request_get_status, Barrier / Ibarrier,
 * Allreduce / Reduce with MPI_SUM, Comm_get_attr(MPI_TAG_UB), Wtime.  Ranks are processes
 * started by `shimrun -n N program args...`.
 *
 * This is baseline tooling: nothing in the framework links against it.
 */
#ifndef ESGD_MPI_SHIM_H
#define ESGD_MPI_SHIM_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef intptr_t MPI_Aint;
struct shim_request;
typedef struct shim_request* MPI_Request;

typedef struct MPI_Status {
  int MPI_SOURCE;
  int MPI_TAG;
  int MPI_ERROR;
  int _cancelled;
  size_t _ucount;
} MPI_Status;

#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_UNDEFINED (-32766)
#define MPI_ANY_SOURCE (-1)
#define MPI_ANY_TAG (-1)
#define MPI_REQUEST_NULL ((MPI_Request)0)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)

#define MPI_CHAR 1
#define MPI_INT 2
#define MPI_FLOAT 3
#define MPI_DOUBLE 4
#define MPI_LONG_LONG 5
#define MPI_BYTE 6

#define MPI_SUM 1
#define MPI_MAX 2
#define MPI_MIN 3

#define MPI_THREAD_SINGLE 0
#define MPI_THREAD_FUNNELED 1
#define MPI_THREAD_SERIALIZED 2
#define MPI_THREAD_MULTIPLE 3

#define MPI_TAG_UB 1

int MPI_Init(int* argc, char*** argv);
int MPI_Init_thread(int* argc, char*** argv, int required, int* provided);
int MPI_Initialized(int* flag);
int MPI_Finalize(void);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_get_attr(MPI_Comm comm, int keyval, void* attribute_val, int* flag);
double MPI_Wtime(void);

int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Test(MPI_Request* req, int* flag, MPI_Status* status);
int MPI_Wait(MPI_Request* req, MPI_Status* status);
int MPI_Testsome(int incount, MPI_Request reqs[], int* outcount, int indices[], MPI_Status statuses[]);
int MPI_Waitsome(int incount, MPI_Request reqs[], int* outcount, int indices[], MPI_Status statuses[]);
int MPI_Cancel(MPI_Request* req);
int MPI_Request_get_status(MPI_Request req, int* flag, MPI_Status* status);

int MPI_Barrier(MPI_Comm comm);
int MPI_Ibarrier(MPI_Comm comm, MPI_Request* req);
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm);
int MPI_Reduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm);

#ifdef __cplusplus
}
#endif
#endif
